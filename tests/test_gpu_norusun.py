"""Norusun on a B200 against the plain CPU restatement (oracle/norusun.py, float64): each mechanism that the design added to
the blocks library alone, then the model through every way of cutting and batching a sequence, the schedulers and the
entry points.  Small made-up configurations and random weights; where random weights would hide a fault (a far key among
hundreds, a sink, the edge of a window or a chunk, the first tokens of a convolution) the inputs are built so that it shows.

Tolerances: relative root-mean-square error of a logits row (mean taken off) below 5e-5 in float32 mode - every product in
true fp32, so only summation order differs.  In bfloat16 mode whole schedules are held to a median of 3e-2 and 95 % of the
rows below 1.5e-1; the float32 run is the sharp test.
"""

import pytest
import torch

from oracle import norusun as O
from extensions_b200.tiny_llm_ext_b200 import blocks
from tiny_llm_b200 import BatchingKvCache, ContinuousBatcher, greedy_generate_ids
from tiny_llm_b200.models import load_model, model_class
from tiny_llm_b200.ragged import RaggedEntry
from tiny_llm_b200.synthetic import norusun_config, save_norusun, synthetic_norusun

pytestmark = pytest.mark.gpu
D64 = torch.float64


@pytest.fixture(scope="module")
def dev(cuda_device):
    return cuda_device


def row_errors(got, want):
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def row_error(got, want):
    return row_errors(got, want).max().item()


def rows_match(got, want, dtype):
    err = row_errors(got, want)
    if dtype == torch.float32:
        return err.max().item() < 5e-5
    return err.median().item() < 3e-2 and err.quantile(0.95).item() < 1.5e-1


def close(got, want, tol):
    got, want = got.double().cpu(), want.double()
    err = (got - want).abs().max().item()
    scale = want.abs().max().item() + 1e-9
    assert err <= tol * scale, (err, scale)


def ids_for(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def info(dev, rows):
    """seq_info rows (first flat token, count, start position, slot)."""
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 4).to(dev)


def in_portions(dev, total, sizes, slot, fn):
    """Run ``fn(lo, hi, seq_info)`` over [0, total) cut into ``sizes`` (the last size repeats); outputs concatenated."""
    out, lo, i = [], 0, 0
    while lo < total:
        n = min(sizes[min(i, len(sizes) - 1)], total - lo)
        out.append(fn(lo, lo + n, info(dev, [0, n, lo, slot])))
        lo, i = lo + n, i + 1
    return torch.cat(out)


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,dim", [(1, 64), (2, 96), (3, 50), (8, 7), (4, 1300)])
def test_residual_streams_write_and_read_in_one_launch(dev, dtype, n, dim):
    g = torch.Generator().manual_seed(n * 1000 + dim)
    rows = 9
    x0, y = torch.randn(rows, dim, generator=g), torch.randn(rows, dim, generator=g)
    mix, w_out, w_in = torch.eye(n) + 0.3 * torch.randn(n, n, generator=g), torch.randn(n, generator=g), torch.randn(n, generator=g)
    bias, gw, eps = torch.randn(dim, generator=g).to(dtype), 1.25, 1e-5
    read = torch.cat([w_in, torch.tensor([gw])]).to(dev)
    write = torch.cat([mix.reshape(-1), w_out]).to(dev)
    xs = torch.full((rows, n, dim), 7.0, device=dev)  # stale numbers: the start must not read them
    h = blocks.streams_step(xs, x0=x0.to(dev), read=read, eps=eps, dtype=dtype)
    want_xs = x0.double()[None].repeat(n, 1, 1)
    norm = lambda u: O.rms_unit(u, eps) * gw
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert torch.equal(xs.cpu(), want_xs.float().transpose(0, 1))
    close(h, norm(O.streams_read(want_xs, w_in.double())), tol)
    h = blocks.streams_step(xs, y=y.to(dev), y_bias=bias.to(dev), write=write, read=read, eps=eps)
    want_xs = O.streams_write(want_xs, y.double() + bias.double(), mix.double(), w_out.double())
    close(xs.transpose(0, 1), want_xs, 2e-6)
    close(h, norm(O.streams_read(want_xs, w_in.double())), tol)
    before = xs.clone()
    assert blocks.streams_step(xs, y=y.to(dev), write=write) is None      # a write alone: the last sublayer of a model
    close(xs.transpose(0, 1), O.streams_write(want_xs, y.double(), mix.double(), w_out.double()), 2e-6)
    total = torch.cat([torch.ones(n), torch.tensor([0.5])]).to(dev)       # the model's norm reads the plain sum, writing nothing
    kept = xs.clone()
    h = blocks.streams_step(xs, read=total, eps=eps, dtype=dtype)
    assert torch.equal(xs, kept) and not torch.equal(xs, before)
    close(h, O.rms_unit(xs.double().cpu().sum(1), eps) * 0.5, tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,n", [(96, 5), (7, 1), (300, 3)])
def test_token_shift_in_portions_batches_and_reused_slots(dev, dtype, dim, n):
    g = torch.Generator().manual_seed(dim)
    T = 80
    h, mu = torch.randn(T, dim, generator=g).to(dtype), torch.rand(n, dim, generator=g).to(dtype)
    before = torch.cat([torch.zeros(1, dim, dtype=D64), h.double()[:-1]])
    want = torch.stack([h.double() + (before - h.double()) * mu[i].double() for i in range(n)])
    state = torch.full((3, dim + 5), 9.0, device=dev)[:, 2 : 2 + dim]     # slots further apart than a row, stale numbers
    hd, mud = h.to(dev), mu.to(dev)
    whole = blocks.shift_mix(hd, mud, seq_info=info(dev, [0, T, 0, 1]), state=state, max_tokens=T)
    close(whole, want, 2e-6 if dtype == torch.float32 else 1e-2)
    assert torch.equal(state[1].cpu(), h[-1].float())
    for sizes in ([1], [2], [1, 2, 3, 33, 1, 40], [32, 1, 31, 2], [64, 16]):
        state.fill_(5.0)
        got = torch.cat([blocks.shift_mix(hd[lo:hi], mud, seq_info=si, state=state, max_tokens=hi - lo) for lo, hi, si in
                         _cuts(dev, T, sizes, 2)], dim=1)
        assert torch.equal(got, whole), sizes
    state.fill_(-3.0)
    blocks.shift_mix(hd[:50], mud, seq_info=info(dev, [0, 50, 0, 0]), state=state, max_tokens=50)
    both = blocks.shift_mix(torch.cat([hd[:20], hd[50:]]), mud, seq_info=info(dev, [[0, 20, 0, 2], [20, 30, 50, 0]]), state=state, max_tokens=30)
    assert torch.equal(both[:, :20], whole[:, :20]) and torch.equal(both[:, 20:], whole[:, 50:])


def _cuts(dev, total, sizes, slot):
    lo, i = 0, 0
    while lo < total:
        n = min(sizes[min(i, len(sizes) - 1)], total - lo)
        yield lo, lo + n, info(dev, [0, n, lo, slot])
        lo, i = lo + n, i + 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels,taps", [(40, 4), (7, 2), (130, 3), (16, 1), (9, 8)])
def test_convolution_with_bias_and_with_the_input_added(dev, dtype, channels, taps):
    g = torch.Generator().manual_seed(channels * 3 + taps)
    T = 90
    x, w, b = torch.randn(T, channels, generator=g).to(dtype), torch.randn(channels, taps, generator=g).to(dtype), torch.randn(channels, generator=g).to(dtype)
    state = torch.full((3, channels, max(taps - 1, 1)), 9.0, device=dev)[:, :, : taps - 1]
    xd, wd, bd = x.to(dev), w.to(dev), b.to(dev)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    for kwargs, want in ((dict(act=1, bias=bd), O.silu(O.causal_conv(x.double(), w.double(), b.double()))),
                         (dict(act=0, add_input=True), x.double() + O.causal_conv(x.double(), w.double()))):
        whole = blocks.short_conv(xd, wd, seq_info=info(dev, [0, T, 0, 1]), state=state, max_tokens=T, **kwargs)
        close(whole, want, tol)
        for sizes in ([1], [2], [1, 2, 3, 33, 1, 40], [64, 26]):
            state.fill_(5.0)
            got = in_portions(dev, T, sizes, 2, lambda lo, hi, si: blocks.short_conv(xd[lo:hi], wd, seq_info=si, state=state, max_tokens=hi - lo, **kwargs))
            assert torch.equal(got, whole), sizes


def wkv_inputs(T, H, dk, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    q, k, v = r(T, H, dk), r(T, H, dk) * dk ** -0.5, r(T, H, dk)
    z, z_bias, bonus = r(T, H * dk), r(H * dk) - 1.5, 0.5 * r(H, dk)
    return [t.to(dtype) for t in (q, k, v)] + [z, z_bias.to(dtype), bonus.to(dtype)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dk", [(2, 16), (3, 40), (1, 64), (2, 33), (4, 1)])
def test_bonus_scan_against_the_recurrence_in_portions_batches_and_reused_slots(dev, dtype, heads, dk):
    T = 150
    q, k, v, z, zb, bonus = wkv_inputs(T, heads, dk, heads * 100 + dk, dtype)
    w = torch.exp(-torch.exp(z.double() + zb.double())).view(T, heads, dk)
    want = O.wkv_sum(q.double(), k.double(), v.double(), w, bonus.double())
    state = torch.full((4, heads, dk, dk), 9.0, device=dev)
    qd, kd, vd, zd, zbd, bd = (t.to(dev) for t in (q, k, v, z, zb, bonus))
    run = lambda lo, hi, si: blocks.decay_scan(qd[lo:hi], kd[lo:hi], vd[lo:hi], zd[lo:hi], zbd, q_scale=1.0, seq_info=si, state=state, max_tokens=hi - lo,
                                               decay_kind=blocks.DECAY_DOUBLE_EXP, bonus=bd)
    walk = in_portions(dev, T, [50], 1, run)                              # portions of up to 64 tokens are single walks
    close(walk, want, 2e-5)
    for sizes in ([1], [2], [1, 2, 3, 33, 1, 40], [64, 64, 22]):
        state.fill_(5.0)
        assert torch.equal(in_portions(dev, T, sizes, 2, run), walk), sizes
    state.fill_(3.0)
    close(run(0, T, info(dev, [0, T, 0, 3])), want, 2e-5)                 # one portion of 150: segments at absolute multiples of 64
    end = state[3].clone()
    state.fill_(3.0)
    close(in_portions(dev, T, [70, 80], 0, run), want, 2e-5)               # segmented portions that start off the grid
    close(state[0], end.double().cpu(), 2e-5)
    # two sequences in one launch: a long one continuing from its slot beside a short new one
    state.fill_(-1.0)
    run(0, 90, info(dev, [0, 90, 0, 2]))
    pick = lambda t: torch.cat([t[90:], t[:20]])
    both = blocks.decay_scan(pick(qd), pick(kd), pick(vd), pick(zd), zbd, q_scale=1.0, seq_info=info(dev, [[0, 60, 90, 2], [60, 20, 0, 1]]), state=state,
                             max_tokens=60, decay_kind=blocks.DECAY_DOUBLE_EXP, bonus=bd)
    assert torch.equal(both[:60], walk[90:]) and torch.equal(both[60:], walk[:20])


def test_a_far_token_is_read_back_through_the_state_and_the_bonus_only_at_its_own_place(dev):
    """Orthogonal keys: token 5 writes value 1 under key e_0 (no decay on that channel); a query for e_0 reads it 700 tokens
    later, through every portion border on the way.  At its own place the token reads bonus * value instead."""
    T, dk = 720, 16
    k = torch.zeros(T, 1, dk)
    k[:, 0, 1] = 1.0          # everybody else writes under e_1
    k[5, 0] = 0.0
    k[5, 0, 0] = 1.0
    v = torch.randn(T, 1, dk, generator=torch.Generator().manual_seed(0))
    q = torch.zeros(T, 1, dk)
    q[5, 0, 0] = q[705, 0, 0] = q[64, 0, 0] = 1.0
    z = torch.zeros(T, dk)
    z[:, 0] = -40.0           # exp(-exp(-40)) = 1: channel 0 never fades
    bonus = torch.full((1, dk), 0.25)
    state = torch.zeros(1, 1, dk, dk, device=dev)
    args = [t.to(dev) for t in (q, k, v, z)]
    for sizes in ([T], [1], [64], [37, 100, 2]):
        got = in_portions(dev, T, sizes, 0, lambda lo, hi, si: blocks.decay_scan(*(a[lo:hi] for a in args), None, q_scale=1.0, seq_info=si, state=state,
                                                                                 max_tokens=hi - lo, decay_kind=blocks.DECAY_DOUBLE_EXP, bonus=bonus.to(dev)))
        close(got[705, 0], v[5, 0], 1e-6)
        close(got[64, 0], v[5, 0], 1e-6)
        close(got[5, 0], 0.25 * v[5, 0], 1e-6)
        assert float(got[6].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,N,P", [(4, 2, 16, 16), (6, 1, 32, 24), (3, 3, 7, 40), (2, 2, 64, 8), (1, 1, 130, 5)])
def test_state_space_scan_against_the_recurrence_with_groups_and_skip(dev, dtype, heads, groups, N, P):
    g = torch.Generator().manual_seed(heads * 7 + N)
    r = lambda *s: torch.randn(*s, generator=g)
    T = 140
    x, B, C = r(T, heads, P).to(dtype), (r(T, groups, N) * N ** -0.5).to(dtype), r(T, groups, N).to(dtype)
    dt_raw, dt_bias, a_log, skip = r(T, heads), (r(heads) - 1.0).to(dtype), (0.5 * r(heads) - 0.5).to(dtype), r(heads).to(dtype)
    dt = O.softplus(dt_raw.double() + dt_bias.double())
    want = O.state_space_sum(x.double(), B.double(), C.double(), dt, torch.exp(a_log.double()), skip.double())
    state = torch.full((3, heads, N, P), 9.0, device=dev)
    xd, Bd, Cd, zd = x.to(dev), B.to(dev), C.to(dev), dt_raw.to(dev)
    run = lambda lo, hi, si: blocks.decay_scan(Cd[lo:hi], Bd[lo:hi], xd[lo:hi], zd[lo:hi], dt_bias.to(dev), q_scale=1.0, seq_info=si, state=state,
                                               max_tokens=hi - lo, decay_kind=blocks.DECAY_STEP, a_log=a_log.to(dev), skip=skip.to(dev))
    walk = in_portions(dev, T, [60], 1, run)
    close(walk, want, 2e-5)
    for sizes in ([1], [2], [3, 1, 50, 2, 64]):
        state.fill_(4.0)
        assert torch.equal(in_portions(dev, T, sizes, 2, run), walk), sizes
    close(run(0, T, info(dev, [0, T, 0, 0])), want, 2e-5)                 # segments


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_a_weight_per_head_and_with_the_gate_before_the_norm(dev, dtype):
    g = torch.Generator().manual_seed(5)
    T, H, dv, eps = 13, 3, 20, 1e-5
    o, w, gate = torch.randn(T, H, dv, generator=g), torch.randn(H * dv, generator=g).to(dtype), torch.randn(T, H * dv, generator=g).to(dtype)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    want = O.rms_unit(o.double(), eps).reshape(T, -1) * w.double() * O.silu(gate.double())
    close(blocks.head_norm_gate(o.to(dev), w.to(dev), eps, gate.to(dev), act=1), want, tol)
    n = (o.double().reshape(T, -1) * O.silu(gate.double())).view(T, H, dv)
    want = O.rms_unit(n, eps).reshape(T, -1) * w.double()
    close(blocks.head_norm_gate(o.to(dev), w.to(dev), eps, gate.to(dev), act=1, gate_first=True), want, tol)
    shared = w[:dv].contiguous()                                                        # the older form: one weight for all heads
    close(blocks.head_norm_gate(o.to(dev), shared.to(dev), eps, None), O.rms_unit(o.double(), eps).reshape(T, -1) * shared.double().repeat(H), tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_and_tanh_rows(dev, dtype):
    g = torch.Generator().manual_seed(6)
    gu = (3 * torch.randn(11, 2 * 37, generator=g)).to(dtype)
    gate, up = gu.double()[:, :37].clamp(max=1.5), gu.double()[:, 37:].clamp(-1.5, 1.5)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    close(blocks.gated_act(gu.to(dev), blocks.ACT_CLAMPED_SWISH, 1.5, 1.702), gate * torch.sigmoid(1.702 * gate) * (up + 1), tol)
    close(blocks.act_rows(gu.to(dev), blocks.ACT_TANH), torch.tanh(gu.double()), tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("heads,kv_heads,dk,dv,dims", [(4, 2, 16, 24, 16), (6, 3, 12, 10, 6), (1, 1, 64, 8, 2), (5, 5, 8, 8, 0), (16, 2, 128, 64, 128)])
def test_norm_over_the_whole_projection_then_rotation_then_the_cache(dev, dtype, interleaved, heads, kv_heads, dk, dv, dims):
    g = torch.Generator().manual_seed(heads * 31 + dk)
    T, eps, base, page = 70, 1e-5, 5e4, 32
    wide = torch.randn(T, heads * dk + kv_heads * (dk + dv) + 5, generator=g).to(dtype)   # q | k | v as columns of one product
    q, k, v = wide[:, : heads * dk], wide[:, heads * dk : (heads + kv_heads) * dk], wide[:, (heads + kv_heads) * dk : (heads + kv_heads) * dk + kv_heads * dv]
    wq, wk = (1 + 0.3 * torch.randn(heads * dk, generator=g)).to(dtype), (1 + 0.3 * torch.randn(kv_heads * dk, generator=g)).to(dtype)
    start = 1000                                                                              # positions far from 0, across a page border
    layout = "interleaved" if interleaved else "half"

    def turned(x, w, n):
        y = (O.rms_unit(x.double(), eps) * w.double()).view(T, n, dk)
        full = torch.zeros(start + T, n, dk, dtype=D64)
        full[start:] = y
        return (O.rotate(full, dims=dims, base=base, layout=layout)[start:] if dims else y).reshape(T, n * dk)

    want_q, want_k = turned(q, wq, heads), turned(k, wk, kv_heads)
    wd = wide.to(dev)
    qd, kd, vd = wd[:, : heads * dk], wd[:, heads * dk : (heads + kv_heads) * dk], wd[:, (heads + kv_heads) * dk : (heads + kv_heads) * dk + kv_heads * dv]
    pages = (start + T) // page + 1
    slab = torch.zeros((pages, page, kv_heads * (dk + dv)), dtype=dtype, device=dev)
    table = torch.arange(pages - 1, -1, -1, dtype=torch.int32, device=dev).reshape(1, -1)    # pages in reverse order
    pos = torch.arange(start, start + T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    blocks.qk_whole_prepare(qd, kd, vd, heads=heads, kv_heads=kv_heads, q_norm=wq.to(dev), k_norm=wk.to(dev), eps=eps, rot_dims=dims, base=base,
                            interleaved=interleaved, tok_pos=pos, tok_seq=seq, block_table=table, slab=slab)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    close(qd, want_q, tol)
    rows = torch.stack([slab[pages - 1 - p // page, p % page] for p in range(start, start + T)])
    close(rows[:, : kv_heads * dk], want_k, tol)
    assert torch.equal(rows[:, kv_heads * dk :].cpu(), v)
    assert torch.equal(kd.cpu(), k) and float(wd[:, -5:].float().sub(wide[:, -5:].float().to(dev)).abs().max()) == 0.0   # keys and neighbours untouched
    if dims:  # the angles read from the step's table instead of evaluated in the kernel: the same numbers
        again, slab2 = wide.to(dev), torch.zeros_like(slab)
        blocks.qk_whole_prepare(again[:, : heads * dk], again[:, heads * dk : (heads + kv_heads) * dk],
                                again[:, (heads + kv_heads) * dk : (heads + kv_heads) * dk + kv_heads * dv], heads=heads, kv_heads=kv_heads, q_norm=wq.to(dev),
                                k_norm=wk.to(dev), eps=eps, rot_dims=dims, base=base, interleaved=interleaved, tok_pos=pos, tok_seq=seq, block_table=table,
                                slab=slab2, rope=blocks.rope_table(pos, dims=dims, base=base))
        assert torch.equal(again, wd) and torch.equal(slab2, slab)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_projection_prepare_gives_a_token_the_same_numbers_in_a_large_step_and_in_a_small_one(dev, dtype):
    """A step of thousands of tokens takes the kernel's warp-per-token form, a small one its CTA-per-token form: bit-identical."""
    g = torch.Generator().manual_seed(77)
    T, heads, kv_heads, dk, dv, dims, page = 2600, 5, 1, 40, 24, 20, 64
    q, k, v = (torch.randn(T, w, generator=g).to(dtype).to(dev) for w in (heads * dk, kv_heads * dk, kv_heads * dv))
    wq, wk = (1 + 0.3 * torch.randn(heads * dk, generator=g)).to(dtype).to(dev), (1 + 0.3 * torch.randn(kv_heads * dk, generator=g)).to(dtype).to(dev)
    pages = -(-T // page)
    table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, -1)
    pos, seq = torch.arange(T, dtype=torch.int32, device=dev), torch.zeros(T, dtype=torch.int32, device=dev)

    def run(cuts):
        qq, slab = q.clone(), torch.zeros((pages, page, kv_heads * (dk + dv)), dtype=dtype, device=dev)
        for lo, hi in cuts:
            blocks.qk_whole_prepare(qq[lo:hi], k[lo:hi], v[lo:hi], heads=heads, kv_heads=kv_heads, q_norm=wq, k_norm=wk, eps=1e-6, rot_dims=dims, base=1e4,
                                    tok_pos=pos[lo:hi], tok_seq=seq[lo:hi], block_table=table, slab=slab)
        return qq, slab

    big_q, big_slab = run([(0, T)])
    small_q, small_slab = run([(lo, min(T, lo + 130)) for lo in range(0, T, 130)])
    assert torch.equal(big_q, small_q) and torch.equal(big_slab, small_slab)
    want = (O.rms_unit(q[:3].double().cpu(), 1e-6) * wq.double().cpu()).view(3, heads, dk)
    close(big_q[:3], O.rotate(want, dims=dims, base=1e4, layout="half").reshape(3, -1), 3e-6 if dtype == torch.float32 else 1e-2)


def fill_cache(dev, rows, page_size, dtype):
    """rows [T, width] -> (slab, block_table) with the tokens' pages in a scrambled order."""
    T, width = rows.shape
    pages = -(-T // page_size)
    order = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(T))[:pages]
    slab = torch.full((pages + 3, page_size, width), 50.0, dtype=dtype, device=dev)     # stale numbers in every unused slot
    for p in range(pages):
        part = rows[p * page_size : (p + 1) * page_size]
        slab[order[p], : part.shape[0]] = part.to(dev)
    return slab, order.to(torch.int32).reshape(1, -1).to(dev)


def tiles_for(dev, first, count, size):
    return torch.tensor([(first + lo, min(size, count - lo), 0) for lo in range(0, count, size)], dtype=torch.int32).to(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,rot,window", [(3, 24, 8, 20), (5, 16, 8, 70), (2, 40, 16, 64), (33, 8, 8, 5)])
def test_latent_attention_with_sinks_at_the_windows_edge(dev, dtype, heads, rank, rot, window):
    """One key carries all the weight: the query of position p asks for position p - window + 1 (just inside) or p - window
    (just outside, where it must find the sink and the rest).  Prompts, single decoded tokens and portions of two."""
    g = torch.Generator().manual_seed(heads + rank)
    T, width, scale = 300, rank + rot, 0.5
    keys = torch.randn(T, width, generator=g)
    keys = 4.0 * keys / keys.norm(dim=1, keepdim=True)
    q = 0.1 * torch.randn(T, heads, width, generator=g)
    for p in range(T):
        for h in range(heads):
            target = p - window + 1 - (h % 2)          # even heads ask just inside the window, odd ones just outside
            if target >= 0:
                q[p, h] = 3.0 * keys[target]
    sink = torch.randn(heads, generator=g)
    keys, q = keys.to(dtype), q.to(dtype)
    want = O.sink_softmax_attention(q.double(), keys.double()[:, None].expand(T, heads, width), keys.double()[:, None, :rank].expand(T, heads, rank),
                                    sink.double(), scale=scale, kind="window", size=window)
    slab, table = fill_cache(dev, keys, 64, dtype)
    kernel, tile = blocks.attention_kernel(dtype, heads, rank, rot, 64)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    qd = q.to(dev)
    tol = 2e-5 if dtype == torch.float32 else 3e-2

    def run(lo, hi):
        out = torch.empty((hi - lo, heads, rank), dtype=dtype, device=dev)
        blocks.latent_attention(qd[lo:hi, :, :rank], qd[lo:hi, :, rank:], slab, table, tiles_for(dev, 0, hi - lo, tile), pos[lo:hi], window=window,
                                scale=scale, out=out, kernel=kernel, max_context=hi, sink=sink.to(dev))
        return out

    close(run(0, T), want, tol)
    close(torch.cat([run(p, p + 1) for p in range(230, 300)]), want[230:], tol)
    close(torch.cat([run(p, p + 2) for p in range(100, 160, 2)]), want[100:160], tol)
    no_sink = torch.empty((T, heads, rank), dtype=dtype, device=dev)
    blocks.latent_attention(qd[:, :, :rank], qd[:, :, rank:], slab, table, tiles_for(dev, 0, T, tile), pos, window=window, scale=scale, out=no_sink,
                            kernel=kernel, max_context=T)
    assert (no_sink.double().cpu() - want).abs().max() > 0.05   # the sink matters in this construction


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dk,dv,chunk", [(4, 2, 16, 24, 24), (6, 3, 32, 32, 150), (3, 3, 8, 8, 64), (5, 1, 12, 20, 7), (2, 1, 64, 128, 33)])
def test_sigmoid_attention_at_the_chunks_edge(dev, dtype, heads, kv_heads, dk, dv, chunk):
    """Weights that do not sum to one: with a strongly negative bias only a key the query points at weighs anything.  The
    query of position p asks for the first position of its chunk (just inside) or the last one of the chunk before (just
    outside: it must read almost nothing)."""
    g = torch.Generator().manual_seed(heads * 10 + dk)
    T, scale = 420, 1.0
    group = heads // kv_heads
    k = torch.randn(T, kv_heads, dk, generator=g)
    k = 4.0 * k / k.norm(dim=2, keepdim=True)
    v = torch.randn(T, kv_heads, dv, generator=g)
    q = 0.05 * torch.randn(T, heads, dk, generator=g)
    for p in range(T):
        for h in range(heads):
            target = p // chunk * chunk - (h % 2)
            if target >= 0:
                q[p, h] = k[target, h // group]
    bias = -8.0 + torch.randn(heads, generator=g)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    want = O.sigmoid_attention(q.double(), k.double().repeat_interleave(group, 1), v.double().repeat_interleave(group, 1), bias.double(), scale=scale,
                               kind="chunk", size=chunk)
    slab, table = fill_cache(dev, torch.cat([k.reshape(T, -1), v.reshape(T, -1)], dim=1), 64, dtype)
    kernel, tile = blocks.paged_attention_kernel(dtype, heads, kv_heads, dk, dv, 64)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    qd = q.to(dev)
    tol = 2e-5 if dtype == torch.float32 else 3e-2

    def run(lo, hi):
        return blocks.paged_attention(qd[lo:hi], slab, table, tiles_for(dev, 0, hi - lo, tile), pos[lo:hi], kv_heads=kv_heads, dv=dv, mask=blocks.MASK_CHUNK,
                                      mask_size=chunk, scale=scale, kernel=kernel, max_context=hi, head_bias=bias.to(dev), weights=blocks.WEIGHTS_SIGMOID)

    assert want.abs().max() > 0.5
    close(run(0, T), want, tol)
    close(torch.cat([run(p, p + 1) for p in range(380, 420)]), want[380:], tol)
    close(torch.cat([run(p, p + 2) for p in range(180, 260, 2)]), want[180:260], tol)


# ---------------------------------------------------------------------------------------------- the model
CONFIGS = {
    # every mixer, two streams, four taps, a layer without a feed-forward
    "mixed": dict(pattern="LdPdWnLd", width=96, vocab=160, wkv_heads=3, wkv_dim=32),
    # what usually differs made equal, or 1: one stream with mixing weights, one tap, one key/value head per head, one state group per head,
    # one norm part, dim = vdim, all of every head rotated, window = chunk = page
    "equal": dict(pattern="PdLdWd", width=64, vocab=97, streams=1, canon_taps=1, heads=2, kv_heads=2, dim=16, vdim=16, rot_dims=16, chunk=64, window=64,
                  lat_heads=2, lat_dim=8, lat_rot=8, lat_vdim=8, kv_rank=16, q_rank=16, ss_heads=2, ss_groups=2, ss_norm_groups=1, ss_state=16, ss_vdim=16,
                  ss_taps=2, wkv_heads=1, wkv_dim=64, ff=64, limit=1.0),
    # sizes that are multiples of nothing: the general attention kernels, three streams, three taps, partial rotation, groups of three
    "odd": dict(pattern="WdPnLd", width=54, vocab=131, streams=3, canon_taps=3, heads=6, kv_heads=2, dim=12, vdim=10, rot_dims=6, chunk=37, window=29,
                lat_heads=5, lat_dim=9, lat_rot=6, lat_vdim=7, kv_rank=21, q_rank=13, ss_heads=6, ss_groups=2, ss_norm_groups=3, ss_state=9, ss_vdim=5,
                ss_taps=3, wkv_heads=2, wkv_dim=27, ff=50, limit=3.5, eps=1e-5),
    # no residual streams and no input convolution at all
    "plain": dict(pattern="LdWnPd", width=64, vocab=120, streams=0, canon_taps=0, wkv_heads=2, wkv_dim=32),
    # no attention layer: a page pool without slabs
    "recurrent": dict(pattern="WdWn", width=48, vocab=90, streams=4, canon_taps=2, wkv_heads=3, wkv_dim=16),
}
_models = {}


def model_and_oracle(dev, name, dtype, max_tokens=None, max_requests=None):
    key = (name, dtype, max_tokens, max_requests)
    if key not in _models:
        config = norusun_config(**CONFIGS[name])
        tensors = synthetic_norusun(config, seed=len(name))
        model = model_class("Norusun").from_checkpoint(config, tensors, dtype=dtype, device=dev, max_tokens=max_tokens, max_requests=max_requests)
        _models[key] = (model, config, tensors)
    return _models[key]


def run_schedule(model, prompts, schedule):
    """``schedule``: steps of [(request, count)]; every position's logits are collected.  Requests end (and give their
    pages and state slot back) with their last token."""
    caches, at, got = {}, {r: 0 for r in prompts}, {r: [] for r in prompts}
    for step in schedule:
        entries = []
        for r, n in step:
            caches.setdefault(r, model.create_kv_cache())
            entries.append(RaggedEntry(prompts[r][at[r] : at[r] + n], caches[r], want=range(n)))
        logits = model.forward_ragged(entries).cpu()
        k = 0
        for r, n in step:
            got[r].append(logits[k : k + n])
            k += n
            at[r] += n
            if at[r] == len(prompts[r]):
                caches.pop(r)[0].release()
    return {r: torch.cat(v) for r, v in got.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_the_plain_model(dev, name, dtype):
    model, config, tensors = model_and_oracle(dev, name, dtype)
    prompt = ids_for(150, config["vocab"], 1)
    want = O.forward(prompt, tensors, config)
    got = run_schedule(model, {"a": prompt}, [[("a", len(prompt))]])["a"]
    assert rows_match(got, want, dtype)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_layers_one_by_one(dev, name):
    """The sum of the streams after every layer (float32 mode), tapped from the model's own step."""
    model, config, tensors = model_and_oracle(dev, name, torch.float32)
    prompt = ids_for(70, config["vocab"], 2)
    want = []
    O.forward(prompt, tensors, config, tap=want)
    cache = model.create_kv_cache()
    model.stream_tap = []
    try:
        model.forward_ragged([RaggedEntry(prompt, cache)])
        assert len(model.stream_tap) == len(want) == len(config["layers"])
        for x, w in zip(model.stream_tap, want):
            close(x, w, 2e-5)
    finally:
        model.stream_tap = None
        cache[0].release()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["mixed", "equal", "odd"])
def test_prefill_then_token_by_token_decoding_across_pages_windows_and_chunks(dev, name, dtype):
    model, config, tensors = model_and_oracle(dev, name, dtype)
    prompt = ids_for(100 + 120, config["vocab"], 3)  # 120 decoded tokens: page borders, windows and chunk edges pass by
    want = O.forward(prompt, tensors, config)
    replays = model.graph_replays
    got = run_schedule(model, {"a": prompt}, [[("a", 100)]] + [[("a", 1)]] * 120)["a"]
    assert rows_match(got, want, dtype)
    assert model.graph_replays - replays >= 110  # single-token steps replay a captured graph from their third step on
    model.use_decode_graph = False
    try:
        eager = run_schedule(model, {"a": prompt}, [[("a", 100)]] + [[("a", 1)]] * 120)["a"]
    finally:
        model.use_decode_graph = None
    assert row_error(eager, got.double()) < 1e-6
    alone = run_schedule(model, {"a": prompt[:40]}, [[("a", 1)]] * 40)["a"]  # the first tokens, one by one from nothing
    assert rows_match(alone, want[:40], dtype)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size_down_to_two(dev, name):
    model, config, tensors = model_and_oracle(dev, name, torch.float32)
    prompt = ids_for(203, config["vocab"], 4)
    want = O.forward(prompt, tensors, config)
    for sizes in ([2] * 20 + [3, 5, 64, 23, 2, 33, 31, 2], [63, 1, 64, 2, 62, 11], [7] * 29, [128, 75]):
        assert sum(sizes) == len(prompt)
        got = run_schedule(model, {"a": prompt}, [[("a", n)] for n in sizes])["a"]
        assert row_error(got, want) < 5e-5, sizes


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_requests_in_one_batch_equal_each_alone_and_pages_and_slots_are_reused(dev, dtype):
    model, config, tensors = model_and_oracle(dev, "mixed", dtype, max_tokens=5 * 64, max_requests=3)
    V = config["vocab"]
    prompts = {"a": ids_for(130, V, 5), "b": ids_for(3, V, 6), "c": ids_for(66, V, 7), "d": ids_for(90, V, 8), "e": ids_for(40, V, 9)}
    want = {r: O.forward(p, tensors, config) for r, p in prompts.items()}
    schedule = [[("a", 60), ("b", 1)], [("a", 2), ("b", 2), ("c", 30)], [("a", 68), ("c", 36)],  # a, b, c end: 3 + 1 + 2 pages come back
                [("d", 64), ("e", 1)], [("d", 1), ("e", 38)], [("d", 25), ("e", 1)]]
    got = run_schedule(model, prompts, schedule)
    for r in prompts:
        assert rows_match(got[r], want[r], dtype), r
    assert model.page_pool.reused_page_allocations > 0 and model.state_pool.reused_slot_allocations > 0
    assert not model.page_pool.used_page_ids and not model.state_pool.used_slots
    if dtype == torch.float32:  # alone, through other pages and slots: the same numbers up to the library products' tile choice
        alone = run_schedule(model, {"d": prompts["d"]}, [[("d", 90)]])["d"]
        assert row_error(alone, got["d"].double()) < 2e-5
    # a fourth live request finds no state slot, a request too long no pages; neither leaves anything behind
    caches = [model.create_kv_cache() for _ in range(4)]
    model.forward_ragged([RaggedEntry([1, 2], c) for c in caches[:3]])
    with pytest.raises(RuntimeError, match="exhausted"):
        model.forward_ragged([RaggedEntry([1], caches[3])])
    with pytest.raises(RuntimeError, match="exhausted"):
        model.forward_ragged([RaggedEntry(list(range(150)) + list(range(60)), caches[0])])
    assert caches[0][0].offset == 2 and caches[3][0].offset == 0
    for c in caches:
        c[0].release()
    assert not model.page_pool.used_page_ids and not model.state_pool.used_slots


@pytest.mark.parametrize("seed", range(10))
def test_random_stacks_and_sizes_in_random_schedules(dev, seed):
    """Layer order, head counts and groups, sizes, streams, taps, windows and chunks drawn at random; the prompt whole, in
    random portions, and as three interleaved requests, in float32."""
    g = torch.Generator().manual_seed(1000 + seed)
    pick = lambda *options: options[int(torch.randint(0, len(options), (1,), generator=g))]
    layers = int(pick(2, 3, 4))
    pattern = "".join(pick("W", "L", "P") + pick("d", "d", "n") for _ in range(layers))
    wkv_heads, wkv_dim = pick((1, 40), (2, 24), (5, 8), (4, 16))
    kv_heads = pick(1, 2, 3)
    ss_groups = pick(1, 2, 3)
    lat_rot = pick(2, 4, 8, 10)
    dim = pick(8, 10, 16, 24)
    width = pick(wkv_heads * wkv_dim, 36, 56)                      # the time-mix heads need not fill the width
    config = norusun_config(pattern=pattern, width=width, vocab=pick(64, 101), streams=pick(0, 1, 2, 3, 5), canon_taps=pick(0, 1, 2, 4, 5),
                            heads=kv_heads * pick(1, 2, 4), kv_heads=kv_heads, dim=dim, vdim=pick(8, 12, 16, 40), chunk=pick(5, 32, 50, 64, 100),
                            rot_dims=pick(2, dim // 2 * 2, dim // 4 * 2 or 2), lat_heads=pick(1, 2, 4, 7), lat_dim=pick(4, 8, 16), lat_rot=lat_rot,
                            lat_vdim=pick(4, 8, 24), kv_rank=pick(8, 14, 32), q_rank=pick(5, 16, 48), window=pick(1, 3, 31, 64, 65, 128),
                            ss_heads=ss_groups * pick(1, 2), ss_groups=ss_groups, ss_norm_groups=pick(1, ss_groups), ss_state=pick(4, 16, 33), ss_vdim=pick(4, 8, 12),
                            ss_taps=pick(1, 2, 4), wkv_heads=wkv_heads, wkv_dim=wkv_dim, ff=pick(24, 64), limit=pick(0.5, 2.0, 7.0), eps=pick(1e-6, 1e-5, 1e-3))
    tensors = synthetic_norusun(config, seed=seed)
    model = model_class("Norusun").from_checkpoint(config, tensors, dtype=torch.float32, device=dev, max_tokens=6 * 64, max_requests=3)
    V = config["vocab"]
    prompts = {"a": ids_for(160, V, seed), "b": ids_for(45, V, seed + 50), "c": ids_for(90, V, seed + 99)}
    want = {r: O.forward(p, tensors, config) for r, p in prompts.items()}
    assert row_error(run_schedule(model, {"a": prompts["a"]}, [[("a", 160)]])["a"], want["a"]) < 5e-5, config
    sizes, left = [], 160
    while left:
        n = min(left, int(pick(1, 2, 2, 3, 7, 30, 64, 70)))
        sizes.append(n)
        left -= n
    assert row_error(run_schedule(model, {"a": prompts["a"]}, [[("a", n)] for n in sizes])["a"], want["a"]) < 5e-5, (config, sizes)
    at, schedule = {r: 0 for r in prompts}, []
    while any(at[r] < len(prompts[r]) for r in prompts):
        step = []
        for r in prompts:
            room = len(prompts[r]) - at[r]
            if room and pick(True, True, False):
                n = min(room, int(pick(1, 1, 2, 5, 40)))
                step.append((r, n))
                at[r] += n
        if step:
            schedule.append(step)
    got = run_schedule(model, prompts, schedule)
    for r in prompts:
        assert row_error(got[r], want[r]) < 1e-4, (r, config)
    assert not model.page_pool.used_page_ids and not model.state_pool.used_slots


def test_long_decoding_keeps_state_and_cache_in_step(dev):
    """500 single-token steps after a two-token prompt (graph replays over growing block tables, windows and chunks sliding
    along), against the plain model."""
    model, config, tensors = model_and_oracle(dev, "mixed", torch.float32)
    prompt = ids_for(502, config["vocab"], 12)
    want = O.forward(prompt, tensors, config)
    got = run_schedule(model, {"a": prompt}, [[("a", 2)]] + [[("a", 1)]] * 500)["a"]
    assert row_error(got, want) < 5e-5


def test_rectangular_call_scheduler_slots_and_offsets(dev):
    model, config, tensors = model_and_oracle(dev, "mixed", torch.float32)
    p0, p1 = ids_for(9, 160, 10), ids_for(5, 160, 11)
    c0, c1 = model.create_kv_cache(), model.create_kv_cache()
    l0 = model(torch.tensor([p0], dtype=torch.int32, device=dev), 0, c0)                 # all rows
    l1 = model(torch.tensor([p1], dtype=torch.int32, device=dev), 0, c1, logits_to_keep=1)
    assert l0.shape == (1, 9, 160) and l1.shape == (1, 1, 160)
    assert row_error(l0[0], O.forward(p0, tensors, config)) < 2e-5
    with pytest.raises(ValueError, match="offset"):
        model(torch.tensor([[1]], dtype=torch.int32, device=dev), 3, c0)
    tables = [BatchingKvCache(max_active_requests=3) for _ in range(model.num_hidden_layers)]
    for t, a, b in zip(tables, c0, c1):
        t.add_request(a, 2)
        t.add_request(b, 0)
    out = model(torch.tensor([[7], [0], [8]], dtype=torch.int32, device=dev), [5, 0, 9], tables, logits_to_keep=1)
    assert out.shape == (3, 1, 160) and float(out[1].abs().max()) == 0.0               # the idle slot
    assert row_error(out[2, 0], O.forward(p0 + [8], tensors, config)[-1]) < 2e-5
    assert row_error(out[0, 0], O.forward(p1 + [7], tensors, config)[-1]) < 2e-5
    for t in tables:
        t.remove_request(0), t.remove_request(2)
    assert not model.page_pool.used_page_ids and not model.state_pool.used_slots


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_entry_points(dev, dtype, tmp_path):
    """greedy_generate_ids and the continuous batcher (mixed steps, 2 slots, 5 requests, pages and state slots reused)
    produce the plain model's greedy tokens; the checkpoint goes through a directory and load_model."""
    config = norusun_config(**CONFIGS["mixed"])
    tensors = synthetic_norusun(config, seed=21)
    save_norusun(config, tensors, tmp_path / "ckpt")
    model = load_model(tmp_path / "ckpt", device=dev, dtype=dtype, max_tokens=6 * 64, max_requests=3)
    prompts = [ids_for(n, 160, 30 + n) for n in (5, 70, 2, 33, 64)]
    new = 30
    want = [O.greedy(p, tensors, config, new) for p in prompts]
    if dtype == torch.float32:
        assert greedy_generate_ids(model, prompts[1], new, device=dev) == want[1]
    batcher = ContinuousBatcher(model, None, prompts, max_seq_len=128, batch_size=2, prefill_step=16, verbose=False, device=dev,
                                max_new_tokens=[new] * len(prompts))
    results = dict(batcher.run())
    got = [[int(t) for t in results[i].split()] for i in range(len(prompts))]
    if dtype == torch.float32:
        assert got == want
    else:  # bf16: the same tokens until a near-tie, at least the first one of most requests
        assert sum(g[:1] == w[:1] for g, w in zip(got, want)) >= len(prompts) - 1
    assert batcher.mixed and batcher.mixed_steps > 0 and model.page_pool.reused_page_allocations > 0 and not model.page_pool.used_page_ids
    assert model.state_pool.reused_slot_allocations > 0 and not model.state_pool.used_slots


def test_trace_program_replays_steps_and_writes_logits(dev, tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    config = norusun_config(**CONFIGS["odd"])
    tensors = synthetic_norusun(config, seed=4)
    save_norusun(config, tensors, tmp_path / "ckpt")
    V = config["vocab"]
    a, b = ids_for(70, V, 1), ids_for(9, V, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:], "want": [0, 3]}, {"id": "b", "tokens": b, "want": [8]}], "end": ["a", "b"]},
             {"step": 2, "entries": [{"id": "c", "tokens": b, "want": [0]}], "end": ["c"]}]
    root = Path(__file__).resolve().parent.parent
    run = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path / "ckpt"), "--dtype", "float32",
                          "--out", str(tmp_path / "out"), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (tmp_path / "out" / "0.f32").exists()
    got = torch.from_numpy(np.fromfile(tmp_path / "out" / "1.f32", dtype="<f4").reshape(3, V))
    wa, wb = O.forward(a, tensors, config), O.forward(b, tensors, config)
    assert row_error(got, torch.stack([wa[66], wa[69], wb[8]])) < 2e-5
    got = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(1, V))
    assert row_error(got, wb[:1]) < 2e-5


def test_command_line_generates_and_batches(dev, tmp_path, capsys):
    from tiny_llm_b200 import cli

    config = norusun_config(**CONFIGS["equal"])
    tensors = synthetic_norusun(config, seed=8)
    save_norusun(config, tensors, tmp_path / "ckpt")
    prompt = ids_for(11, 97, 5)
    want = O.greedy(prompt, tensors, config, 6)
    assert cli.main(["generate", "--model", str(tmp_path / "ckpt"), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                     "--max-new-tokens", "6"]) == 0
    assert [int(t) for t in capsys.readouterr().out.split()] == want
    assert cli.main(["batch", "--model", str(tmp_path / "ckpt"), "--dtype", "float32", "--quiet", "--batch-size", "2", "--prefill-step", "4",
                     "--max-new-tokens", "6", "--prompt-ids", ";".join(",".join(map(str, ids_for(n, 97, n))) for n in (11, 3, 7))]) == 0
    out = capsys.readouterr().out
    assert out.count("--- request") == 3
    first = out.split("--- request 0\n")[1].split("\n")[0]
    assert [int(t) for t in first.split()] == O.greedy(ids_for(11, 97, 11), tensors, config, 6)
    assert cli.main(["generate", "--synthetic", "norusun:PdWn", "--prompt-ids", "5,17,3", "--max-new-tokens", "4"]) == 0
    assert len(capsys.readouterr().out.split()) == 4
