"""ctypes binding of ``libtiny_llm_b200_blocks.so`` (C ABI: ``include/tiny_llm_b200_blocks.h``): row-wise norms over
an fp32 residual stream, rotary positions, the paged latent cache, latent attention over ragged batches, gated
activations and the mixture-of-experts kernels.  Arguments are contiguous CUDA ``torch.Tensor`` s (strided where the
function says so); every call enqueues on the current stream.  There is no CPU path.

The library is built on first use when it is missing (a handful of translation units, compiled side by side)."""

from __future__ import annotations

import ctypes
import importlib.util
import os
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB_NAME = "libtiny_llm_b200_blocks.so"
_lib = None

_VP, _I, _F, _D, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_double, ctypes.c_longlong

_SIGNATURES = {
    "tlb_abi_version": (_I, []),
    "tlb_last_error": (ctypes.c_char_p, []),
    "tlb_launch_count": (_LL, []),
    "tlb_embed_rows": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _VP]),
    "tlb_norm_residual": (_I, [_VP, _I, _VP, _F, _VP, _F, _VP, _VP, _I, _I, _I, _VP]),
    "tlb_rope_rows": (_I, [_VP, _LL, _LL, _I, _I, _I, _I, _D, _D, _VP, _I, _I, _VP]),
    "tlb_rope_table": (_I, [_VP, _I, _I, _D, _D, _VP, _VP, _VP]),
    "tlb_latent_append": (_I, [_VP, _VP, _F, _I, _I, _I, _I, _D, _VP, _VP, _VP, _I, _I, _I, _VP, _I, _I, _VP]),
    "tlb_latent_prepare": (_I, [_VP, _LL, _VP, _F, _I, _I, _I, _I, _D, _VP, _VP, _VP, _I, _I, _I, _VP, _VP, _LL, _I, _I, _I, _I, _I, _VP]),
    "tlb_latent_attention": (_I, [_VP, _LL, _LL, _VP, _LL, _LL, _VP, _I, _I, _I, _I, _VP, _I, _VP, _I, _VP, _I, _I, _F, _VP, _LL, _LL, _VP, _I, _VP]),
    "tlb_latent_attention_mma_tile_tokens": (_I, [_I]),
    "tlb_latent_attention_mma_supported": (_I, [_I, _I, _I]),
    "tlb_latent_attention_mma": (_I, [_VP, _LL, _LL, _VP, _LL, _LL, _VP, _I, _I, _I, _I, _VP, _I, _VP, _I, _VP, _I, _I, _F, _VP, _LL, _LL, _I, _VP,
                                      ctypes.c_size_t, _VP, _VP]),
    "tlb_latent_attention_mma_workspace": (ctypes.c_size_t, [_I, _I, _I, _I]),
    "tlb_gated_act": (_I, [_VP, _VP, _I, _I, _I, _F, _F, _I, _VP]),
    "tlb_streams_step": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _F, _VP, _I, _I, _I, _I, _VP]),
    "tlb_shift_mix": (_I, [_VP, _LL, _VP, _I, _I, _VP, _I, _I, _VP, _LL, _I, _VP, _LL, _I, _VP]),
    "tlb_moe_route": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP, _F, _VP, _VP, _I, _VP]),
    "tlb_moe_up": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _VP, _I, _VP]),
    "tlb_moe_scale_rows": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _VP]),
    "tlb_add_norm": (_I, [_VP, _VP, _I, _VP, _VP, _F, _VP, _I, _I, _I, _VP]),
    "tlb_norm_mix2": (_I, [_VP, _VP, _VP, _VP, _F, _F, _VP, _I, _I, _I, _VP]),
    "tlb_paged_attention_tile_tokens": (_I, [_I, _I]),
    "tlb_paged_attention": (_I, [_VP, _LL, _LL, _VP, _I, _I, _I, _I, _I, _I, _VP, _I, _VP, _I, _VP, _I, _I, _F, _F, _I, _VP, _LL, _VP, _LL, _LL, _VP, _I, _I,
                                 _VP]),
    "tlb_paged_attention_mma_tile_tokens": (_I, [_I, _I]),
    "tlb_paged_attention_mma_supported": (_I, [_I, _I, _I, _I]),
    "tlb_paged_attention_mma": (_I, [_VP, _LL, _LL, _VP, _I, _I, _I, _I, _I, _I, _VP, _I, _VP, _I, _VP, _I, _I, _F, _F, _I, _VP, _LL, _VP, _LL, _LL, _I, _VP,
                                     ctypes.c_size_t, _VP, _I, _VP]),
    "tlb_paged_attention_mma_workspace": (ctypes.c_size_t, [_I, _I, _I, _I, _I]),
    "tlb_kv_prepare": (_I, [_VP, _LL, _LL, _I, _VP, _VP, _LL, _LL, _VP, _LL, _LL, _I, _I, _I, _VP, _F, _VP, _VP, _VP, _I, _I, _I, _VP, _I, _I, _VP]),
    "tlb_qk_whole_prepare": (_I, [_VP, _LL, _I, _VP, _VP, _LL, _VP, _LL, _I, _I, _I, _VP, _F, _I, _I, _D, _VP, _VP, _VP, _I, _I, _I, _VP, _VP, _VP, _I, _I, _VP]),
    "tlb_decay_scan_workspace": (ctypes.c_size_t, [_I, _I, _I, _I, _I]),
    "tlb_decay_scan": (_I, [_VP, _LL, _LL, _VP, _LL, _LL, _VP, _LL, _LL, _VP, _LL, _VP, _F, _VP, _VP, _VP, _I, _I, _F, _I, _I, _I, _VP, _I, _I, _VP, _LL, _I,
                            _VP, _VP, ctypes.c_size_t, _I, _VP, _VP, _I, _VP, _I, _VP]),
    "tlb_delta_scan_workspace": (ctypes.c_size_t, [_I, _I, _I, _I, _I]),
    "tlb_delta_scan": (_I, [_VP, _LL, _LL, _VP, _LL, _LL, _VP, _LL, _LL, _VP, _LL, _VP, _I, _LL, _I, _VP, _VP, _F, _F, _I, _I, _I, _I, _VP, _I, _I, _VP, _LL,
                            _I, _VP, _VP, ctypes.c_size_t, _I, _VP]),
    "tlb_short_conv": (_I, [_VP, _LL, _VP, _VP, _I, _I, _I, _I, _VP, _I, _I, _VP, _LL, _I, _VP, _I, _VP]),
    "tlb_act_rows": (_I, [_VP, _VP, _I, _I, _I, _I, _VP]),
    "tlb_softcap_rows": (_I, [_VP, _I, _I, _F, _VP]),
    "tlb_cast_rows": (_I, [_VP, _VP, _LL, _I, _I, _I, _VP]),
    "tlb_head_norm_gate": (_I, [_VP, _VP, _F, _VP, _LL, _I, _VP, _I, _I, _I, _I, _I, _I, _VP]),
    "tlb_moe_max_rows": (_LL, [_I, _I, _I, _I]),
    "tlb_moe_sort": (_I, [_VP, _I, _I, _I, _I, _VP, _VP, _VP, _VP]),
    "tlb_moe_gate_up": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _VP, _I, _VP]),
    "tlb_moe_down": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP, _I, _VP]),
    "tlb_moe_combine": (_I, [_VP, _VP, _VP, _VP, _I, _VP, _VP, _I, _I, _I, _I, _VP]),
    "tlb_argmax_rows": (_I, [_VP, _VP, _I, _I, _VP]),
}
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

ABI_VERSION = 5
ATTENTION_TILE_TOKENS = 4
MOE_TILE_ROWS = 32
ACT_SILU, ACT_GELU_TANH, ACT_RELU_SQUARED, ACT_CLAMPED_SWISH, ACT_TANH = 0, 1, 2, 3, 4
WEIGHTS_SOFTMAX, WEIGHTS_SIGMOID = 0, 1
DECAY_SIGMOID, DECAY_DOUBLE_EXP, DECAY_STEP = 0, 2, 3
MASK_CAUSAL, MASK_WINDOW, MASK_CHUNK = 0, 1, 2
SCORE_SOFTMAX, SCORE_SIGMOID, SCORE_SOFTMAX_ALL = 0, 1, 2
_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 2}


def _build() -> Path:
    script = _HERE.parent.parent / "csrc" / "build.py"
    spec = importlib.util.spec_from_file_location("tiny_llm_b200_build", script)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.build_blocks()


def load_library(path: str | os.PathLike | None = None) -> None:
    """Load the library, compiling it first when the in-tree file is missing (``ImportError`` if that fails)."""
    global _lib
    candidate = Path(path) if path is not None else _HERE / _LIB_NAME
    if not candidate.exists():
        if path is not None:
            raise ImportError(f"{candidate} not found")
        try:
            candidate = _build()
        except Exception as exc:  # no nvcc, read-only tree, compile error
            raise ImportError(f"{candidate} is not built and could not be compiled: {exc}") from exc
    lib = ctypes.CDLL(str(candidate))
    lib.tlb_abi_version.restype = _I
    if lib.tlb_abi_version() != ABI_VERSION:  # a library built from other sources: calling it with these signatures would crash
        if path is not None:
            raise ImportError(f"{candidate} has ABI {lib.tlb_abi_version()}, this binding needs {ABI_VERSION}")
        try:
            candidate = _build()
        except Exception as exc:
            raise ImportError(f"{candidate} is out of date and could not be rebuilt: {exc}") from exc
        lib = ctypes.CDLL(str(candidate))
        lib.tlb_abi_version.restype = _I
        if lib.tlb_abi_version() != ABI_VERSION:
            raise ImportError(f"{candidate} has ABI {lib.tlb_abi_version()}, this binding needs {ABI_VERSION}")
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib


def library():
    if _lib is None:
        load_library(os.environ.get("TL_BLOCKS_LIB") or None)
    return _lib


def launch_count() -> int:
    return int(library().tlb_launch_count())


def _code(t: torch.dtype) -> int:
    if t not in _DTYPE_CODE:
        raise RuntimeError(f"blocks: dtype {t} is not float32 or bfloat16")
    return _DTYPE_CODE[t]


def _gpu(op: str, *tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(f"{op}: the blocks extension is GPU-only")


def _contig(op: str, *tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise RuntimeError(f"{op}: arguments must be contiguous")


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def _stream(ref: torch.Tensor) -> int:
    return torch.cuda.current_stream(ref.device).cuda_stream


def _check(code: int) -> None:
    if code != 0:
        raise RuntimeError(library().tlb_last_error().decode() or f"tiny_llm_b200_blocks error {code}")


def embed_rows(ids: torch.Tensor, table: torch.Tensor):
    """-> (x32 [T, D] fp32 residual stream, h [T, D] in the table's dtype)."""
    _gpu("embed_rows", ids, table)
    _contig("embed_rows", ids, table)
    if ids.dtype != torch.int32 or ids.dim() != 1 or table.dim() != 2:
        raise RuntimeError("embed_rows: ids must be int32 [T] and table [vocab, dim]")
    T, (V, D) = ids.numel(), table.shape
    x32 = torch.empty((T, D), dtype=torch.float32, device=table.device)
    h = torch.empty((T, D), dtype=table.dtype, device=table.device)
    _check(library().tlb_embed_rows(_ptr(ids), _ptr(table), _ptr(x32), _ptr(h), T, V, D, _code(table.dtype), _stream(table)))
    return x32, h


def norm_residual(y, weight, eps: float, *, weight_offset: float = 0.0, scale=None, residual=None, want_h: bool = True):
    """RMS norm of ``y [rows, dim]`` (fp32 or the weight's dtype) times ``weight + weight_offset`` (times ``scale``);
    with ``residual`` (fp32, updated in place) the result is added to it.  Returns the (new residual, or the norm)
    rounded to the weight's dtype, or None when ``want_h`` is false."""
    _gpu("norm_residual", y, weight, scale, residual)
    _contig("norm_residual", y, weight, scale, residual)
    rows, dim = y.shape
    if y.dtype not in (torch.float32, weight.dtype):
        raise RuntimeError("norm_residual: y must be float32 or the weight's dtype")
    if weight.shape != (dim,) or (scale is not None and (scale.shape != (dim,) or scale.dtype != weight.dtype)):
        raise RuntimeError("norm_residual: weight / scale must be [dim] of one dtype")
    if residual is not None and (residual.dtype != torch.float32 or residual.shape != y.shape):
        raise RuntimeError("norm_residual: residual must be float32 of y's shape")
    if residual is None and not want_h:
        raise RuntimeError("norm_residual: nothing to write")
    h = torch.empty((rows, dim), dtype=weight.dtype, device=y.device) if want_h else None
    _check(library().tlb_norm_residual(_ptr(y), int(y.dtype == torch.float32), _ptr(weight), float(weight_offset), _ptr(scale), float(eps),
                                       _ptr(residual), _ptr(h), rows, dim, _code(weight.dtype), _stream(y)))
    return h


def rope_rows(x: torch.Tensor, tok_pos: torch.Tensor, *, heads: int, head_stride: int, first: int, dims: int, base: float, interleaved: bool,
              factor: float = 1.0):
    """Rotate, in place, ``dims`` entries from ``first`` in each of ``heads`` heads of every row of ``x [rows, *]``;
    ``factor`` divides every frequency (linear scaling of the positions)."""
    _gpu("rope_rows", x, tok_pos)
    if x.dim() != 2 or x.stride(1) != 1 or tok_pos.dtype != torch.int32 or tok_pos.numel() != x.shape[0]:
        raise RuntimeError("rope_rows: x must be [rows, n] with unit inner stride and tok_pos int32 [rows]")
    if first + dims > head_stride or (heads - 1) * head_stride + first + dims > x.shape[1]:
        raise RuntimeError("rope_rows: rotated entries fall outside the row")
    _check(library().tlb_rope_rows(_ptr(x), x.stride(0), head_stride, first, heads, dims, int(interleaved), float(base), float(factor), _ptr(tok_pos),
                                   x.shape[0], _code(x.dtype), _stream(x)))
    return x


def rope_table(tok_pos: torch.Tensor, *, dims: int, base: float, factor: float = 1.0):
    """-> (cos, sin) fp32 ``[rows, dims // 2]`` of ``tok_pos * base^(-2i/dims) / factor``, for kernels that rotate in fp32."""
    _gpu("rope_table", tok_pos)
    if tok_pos.dtype != torch.int32 or tok_pos.dim() != 1 or not tok_pos.is_contiguous() or dims <= 0 or dims % 2:
        raise RuntimeError("rope_table: tok_pos must be contiguous int32 [rows] and dims even")
    rows = tok_pos.numel()
    cs = torch.empty((rows, dims // 2), dtype=torch.float32, device=tok_pos.device)
    sn = torch.empty_like(cs)
    _check(library().tlb_rope_table(_ptr(tok_pos), rows, int(dims), float(base), float(factor), _ptr(cs), _ptr(sn), _stream(tok_pos)))
    return cs, sn


def latent_append(down, norm_weight, eps, *, rank, rot_dims, interleaved, base, tok_pos, tok_seq, block_table, slab):
    """Norm the latent, rotate the shared key part and store both at every token's slot of ``slab [P, page, rank+rot]``."""
    _gpu("latent_append", down, norm_weight, tok_pos, tok_seq, block_table, slab)
    _contig("latent_append", down, norm_weight, tok_pos, tok_seq, block_table, slab)
    T, width = down.shape
    P, page_size, w2 = slab.shape
    if w2 != width or slab.dtype != down.dtype or norm_weight.dtype != down.dtype or norm_weight.numel() != rank:
        raise RuntimeError("latent_append: slab / weight do not match the projection")
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or tok_pos.numel() != T or tok_seq.numel() != T:
        raise RuntimeError("latent_append: bad metadata")
    _check(library().tlb_latent_append(_ptr(down), _ptr(norm_weight), float(eps), rank, width - rank, rot_dims, int(interleaved), float(base),
                                       _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), block_table.shape[1], P, page_size, _ptr(slab), T,
                                       _code(down.dtype), _stream(down)))


def latent_prepare(qd, norm_weight, eps, *, heads, dim, rot_dim, rank, rot_dims, interleaved, base, tok_pos, tok_seq, block_table, slab):
    """One launch after a fused q|dkv projection ``qd [T, heads * (dim + rot_dim) + rank + rot_dim]``: rotate the rotated
    part of every query head in place, norm the latent, rotate the shared key part and store both in ``slab``."""
    _gpu("latent_prepare", qd, norm_weight, tok_pos, tok_seq, block_table, slab)
    _contig("latent_prepare", qd, norm_weight, tok_pos, tok_seq, block_table, slab)
    T, total = qd.shape
    P, page_size, width = slab.shape
    q_width = heads * (dim + rot_dim)
    if total != q_width + width or width != rank + rot_dim or slab.dtype != qd.dtype or norm_weight.dtype != qd.dtype or norm_weight.numel() != rank:
        raise RuntimeError("latent_prepare: projection, slab and weight do not match")
    es = qd.element_size()
    _check(library().tlb_latent_prepare(qd.data_ptr() + q_width * es, total, _ptr(norm_weight), float(eps), rank, rot_dim, rot_dims, int(interleaved),
                                        float(base), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), block_table.shape[1], P, page_size, _ptr(slab),
                                        _ptr(qd), total, heads, dim + rot_dim, dim, T, _code(qd.dtype), _stream(qd)))


def latent_prepare_parts(q, down, norm_weight, eps, *, heads, dim, rot_dim, rank, rot_dims, interleaved, base, tok_pos, tok_seq, block_table, slab):
    """``latent_prepare`` for queries and down projection that are separate matrices (views with unit inner stride):
    ``q [T, heads * (dim + rot_dim)]`` rotated in place, ``down [T, rank + rot_dim]`` normed, rotated and stored."""
    _gpu("latent_prepare", q, down, norm_weight, tok_pos, tok_seq, block_table, slab)
    _contig("latent_prepare", norm_weight, tok_pos, tok_seq, block_table, slab)
    T = q.shape[0]
    P, page_size, width = slab.shape
    if q.shape != (T, heads * (dim + rot_dim)) or down.shape != (T, width) or width != rank + rot_dim or q.stride(1) != 1 or down.stride(1) != 1:
        raise RuntimeError("latent_prepare: queries, down projection and slab do not match")
    if not (slab.dtype == q.dtype == down.dtype == norm_weight.dtype) or norm_weight.numel() != rank:
        raise RuntimeError("latent_prepare: one dtype, and a weight of [rank]")
    _check(library().tlb_latent_prepare(_ptr(down), down.stride(0), _ptr(norm_weight), float(eps), rank, rot_dim, rot_dims, int(interleaved), float(base),
                                        _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), block_table.shape[1], P, page_size, _ptr(slab), _ptr(q),
                                        q.stride(0), heads, dim + rot_dim, dim, T, _code(q.dtype), _stream(q)))


def attention_kernel(dtype, heads: int, rank: int, rot: int, page_size: int) -> tuple[str, int]:
    """Which latent-attention kernel serves these sizes, and the most tokens one entry of its ``tiles`` may hold:
    ``("mma", 32 // min(heads, 32))`` for a bf16 cache the tensor-core kernel can take (32 query rows per CTA), else
    ``("general", 4)`` (fp32 cache, odd widths; TL_LATENT_MMA=0 forces it)."""
    if dtype == torch.bfloat16 and _mma_ok(rank, rot, page_size):
        return "mma", int(library().tlb_latent_attention_mma_tile_tokens(heads))
    return "general", ATTENTION_TILE_TOKENS


_SM_COUNT: dict = {}


def attention_splits(num_ctas: int, max_context: int, device) -> int:
    """Into how many CTAs to cut every tile's key range: 1 while the launch fills the GPU by itself, else enough to give
    every SM a CTA, each with at least two 64-key tiles."""
    key = torch.device(device)
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(key).multi_processor_count
    sms = _SM_COUNT[key]
    if num_ctas * 2 > sms:
        return 1
    return max(1, min(sms // num_ctas, max_context // 128, 32))


def latent_attention(q_lat, q_rot, slab, block_table, tiles, tok_pos, *, window: int, scale: float, out, kernel: str = "general", max_context: int = 0,
                     sink=None):
    """``q_lat [T, H, rank]``, ``q_rot [T, H, rot]`` and ``out [T, H, rank]`` are views with arbitrary token / head strides
    and unit inner stride; ``tiles [n, 3]`` int32 (first token, count, block-table row) cut for the tile size that
    ``attention_kernel`` gives beside the kernel's name.  ``max_context`` (the longest sequence of the step, 0 = unknown)
    lets the tensor-core kernel split the key range over several CTAs when the launch alone would leave SMs idle.
    ``sink`` (fp32 ``[H]``): one more term ``exp(sink[h])`` in head h's softmax denominator, without a key or a value."""
    _gpu("latent_attention", q_lat, q_rot, slab, block_table, tiles, tok_pos, out, sink)
    if sink is not None and (sink.dtype != torch.float32 or sink.shape != (q_lat.shape[1],) or not sink.is_contiguous()):
        raise RuntimeError("latent_attention: sink must be float32 [H]")
    _contig("latent_attention", slab, block_table, tiles, tok_pos)
    T, H, rank = q_lat.shape
    P, page_size, width = slab.shape
    rot = width - rank
    if q_rot.shape != (T, H, rot) or out.shape != (T, H, rank) or q_lat.stride(2) != 1 or q_rot.stride(2) != 1 or out.stride(2) != 1:
        raise RuntimeError("latent_attention: query / output shapes do not match the cache")
    if not (q_lat.dtype == q_rot.dtype == slab.dtype == out.dtype):
        raise RuntimeError("latent_attention: one dtype for queries, cache and output")
    lib = library()
    if kernel == "mma":
        if slab.dtype != torch.bfloat16:
            raise RuntimeError("latent_attention: the tensor-core kernel takes a bfloat16 cache")
        reach = min(max_context, int(window)) if window else max_context  # keys a query can see at most
        rows = int(lib.tlb_latent_attention_mma_tile_tokens(1))  # query rows per CTA
        splits = attention_splits(tiles.shape[0] * -(-H // rows), reach, slab.device) if reach else 1
        nbytes = int(lib.tlb_latent_attention_mma_workspace(tiles.shape[0], H, rank, splits))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=slab.device) if nbytes else None
        _check(lib.tlb_latent_attention_mma(_ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), q_rot.stride(0), q_rot.stride(1), _ptr(slab), P,
                                            page_size, rank, rot, _ptr(block_table), block_table.shape[1], _ptr(tiles), tiles.shape[0], _ptr(tok_pos),
                                            H, int(window or 0), float(scale), _ptr(out), out.stride(0), out.stride(1), splits, _ptr(ws), nbytes,
                                            _ptr(sink), _stream(slab)))
        return out
    if kernel != "general":
        raise RuntimeError(f"latent_attention: unknown kernel {kernel!r}")
    _check(lib.tlb_latent_attention(_ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), q_rot.stride(0), q_rot.stride(1), _ptr(slab), P,
                                    page_size, rank, rot, _ptr(block_table), block_table.shape[1], _ptr(tiles), tiles.shape[0], _ptr(tok_pos),
                                    H, int(window or 0), float(scale), _ptr(out), out.stride(0), out.stride(1), _ptr(sink), _code(slab.dtype), _stream(slab)))
    return out


def _mma_ok(rank: int, rot: int, page_size: int) -> bool:
    return os.environ.get("TL_LATENT_MMA", "1") != "0" and bool(library().tlb_latent_attention_mma_supported(rank, rot, page_size))


def gated_act(gate_up: torch.Tensor, act: int, limit: float = 0.0, slope: float = 1.0) -> torch.Tensor:
    """``act(gate) * up`` of ``[rows, 2 * width]`` (gate columns first).  ``ACT_CLAMPED_SWISH``: ``g = min(gate, limit)``,
    ``u = clamp(up, -limit, limit)``, ``g sigmoid(slope g) (u + 1)``."""
    _gpu("gated_act", gate_up)
    _contig("gated_act", gate_up)
    rows, two = gate_up.shape
    out = torch.empty((rows, two // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(library().tlb_gated_act(_ptr(gate_up), _ptr(out), rows, two // 2, act, float(limit), float(slope), _code(gate_up.dtype), _stream(gate_up)))
    return out


def moe_route(h, router_w, router_b, top: int, scoring: int = SCORE_SOFTMAX, choice_bias=None, weight_scale: float = 1.0):
    """-> (expert ids int32 [T, top], weights fp32 [T, top]): softmax over the chosen logits, each one's sigmoid, or
    (``SCORE_SOFTMAX_ALL``) a softmax over all outputs, chosen by score + ``choice_bias``, the chosen scores renormalised
    and times ``weight_scale``."""
    _gpu("moe_route", h, router_w, router_b, choice_bias)
    _contig("moe_route", h, router_w, router_b, choice_bias)
    if choice_bias is not None and (choice_bias.dtype != h.dtype or choice_bias.numel() != router_w.shape[0]):
        raise RuntimeError("moe_route: choice_bias must be [experts] of the activations' dtype")
    T, D = h.shape
    E = router_w.shape[0]
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    gate = torch.empty((T, top), dtype=torch.float32, device=h.device)
    _check(library().tlb_moe_route(_ptr(h), _ptr(router_w), _ptr(router_b), T, D, E, top, int(scoring), _ptr(choice_bias), float(weight_scale), _ptr(idx),
                                   _ptr(gate), _code(h.dtype), _stream(h)))
    return idx, gate


def moe_experts(h, idx, gate, w_gate, w_up, w_down, act: int, shared=None, scale_input: bool = False, identity: bool = False) -> torch.Tensor:
    """Sum of the chosen experts' feed-forwards (+ ``shared [T, D]``) -> fp32 ``[T, D]``.  ``w_up [E, ff, D]``,
    ``w_down [E, D, ff]``; with ``w_gate [E, ff, D]`` an expert is ``down(act(gate x) * (up x))``, without it
    ``down(act(up x))``.  The router's weight multiplies the expert's output, or, ``scale_input``, its input ``x``
    (rounded to the compute dtype).  ``identity``: ids from ``E`` up name identity experts, whose output is the token itself."""
    _gpu("moe_experts", h, idx, gate, w_gate, w_up, w_down, shared)
    _contig("moe_experts", h, idx, gate, w_gate, w_up, w_down, shared)
    lib = library()
    T, D = h.shape
    E, ff, _ = w_up.shape
    top = idx.shape[1]
    # 64-row expert tiles once the average expert gets that many rows (tensor-core kernels only: bf16, widths % 8 == 0)
    rows = 64 if (h.dtype == torch.bfloat16 and D % 8 == 0 and ff % 8 == 0 and T * top >= 64 * E) else MOE_TILE_ROWS
    max_rows = int(lib.tlb_moe_max_rows(T, top, E, rows))
    dev, code, st = h.device, _code(h.dtype), _stream(h)
    sorted_pair = torch.empty(max_rows, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(max_rows // rows, dtype=torch.int32, device=dev)
    counters = torch.empty(2, dtype=torch.int32, device=dev)
    inter = torch.empty((max_rows, ff), dtype=h.dtype, device=dev)
    pair_out = torch.empty((T * top, D), dtype=torch.float32, device=dev)
    y = torch.empty((T, D), dtype=torch.float32, device=dev)
    _check(lib.tlb_moe_sort(_ptr(idx), T, top, E, rows, _ptr(sorted_pair), _ptr(tile_expert), _ptr(counters), st))
    rows_in, per_pair = h, 0
    if scale_input:
        rows_in, per_pair = torch.empty((T * top, D), dtype=h.dtype, device=dev), 1
        _check(lib.tlb_moe_scale_rows(_ptr(h), _ptr(gate), _ptr(rows_in), T, top, D, code, st))
    if w_gate is not None:
        if per_pair:
            raise RuntimeError("moe_experts: gated experts take the router's weight on their output")
        _check(lib.tlb_moe_gate_up(_ptr(h), _ptr(w_gate), _ptr(w_up), _ptr(sorted_pair), _ptr(tile_expert), _ptr(counters), T, top, E, rows, D, ff, act,
                                   _ptr(inter), code, st))
    else:
        _check(lib.tlb_moe_up(_ptr(rows_in), _ptr(w_up), _ptr(sorted_pair), _ptr(tile_expert), _ptr(counters), T, top, E, rows, D, ff, act, per_pair,
                              _ptr(inter), code, st))
    _check(lib.tlb_moe_down(_ptr(inter), _ptr(w_down), _ptr(sorted_pair), _ptr(tile_expert), _ptr(counters), T, top, E, rows, D, ff, _ptr(pair_out), code, st))
    _check(lib.tlb_moe_combine(_ptr(pair_out), None if scale_input else _ptr(gate), _ptr(shared), _ptr(idx) if identity else None, E,
                               _ptr(h) if identity else None, _ptr(y), T, top, D, code, st))
    return y


def add_norm(residual: torch.Tensor, a: torch.Tensor, b: torch.Tensor | None, weight: torch.Tensor | None, eps: float):
    """``residual += a (+ b)`` (all fp32 ``[rows, dim]``, in place; ``a`` may be one row ``[dim]`` for all); with ``weight``
    also returns the RMS norm of the new residual times ``weight``, rounded to the weight's dtype."""
    _gpu("add_norm", residual, a, b, weight)
    _contig("add_norm", residual, a, b, weight)
    rows, dim = residual.shape
    a_row = a.dim() == 1
    if residual.dtype != torch.float32 or a.dtype != torch.float32 or a.shape != (residual.shape[1:] if a_row else residual.shape) or (b is not None and (b.dtype != torch.float32 or b.shape != residual.shape)):
        raise RuntimeError("add_norm: residual and addends must be float32 of one shape")
    h = None if weight is None else torch.empty((rows, dim), dtype=weight.dtype, device=residual.device)
    code = _code(weight.dtype) if weight is not None else 0
    _check(library().tlb_add_norm(_ptr(residual), _ptr(a), int(a_row), _ptr(b), _ptr(weight), float(eps), _ptr(h), rows, dim, code, _stream(residual)))
    return h


def norm_mix2(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, coef: float, eps: float) -> torch.Tensor:
    """``coef * (rms_norm(a) * wa + rms_norm(b) * wb)``: fp32 ``[rows, dim]`` in and out."""
    _gpu("norm_mix2", a, wa, b, wb)
    _contig("norm_mix2", a, wa, b, wb)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape != b.shape or wa.dtype != wb.dtype:
        raise RuntimeError("norm_mix2: a and b must be float32 of one shape, the weights of one dtype")
    y = torch.empty_like(a)
    _check(library().tlb_norm_mix2(_ptr(a), _ptr(wa), _ptr(b), _ptr(wb), float(coef), float(eps), _ptr(y), a.shape[0], a.shape[1], _code(wa.dtype), _stream(a)))
    return y


def paged_attention_kernel(dtype, heads: int, kv_heads: int, dk: int, dv: int, page_size: int) -> tuple[str, int]:
    """Which grouped-query attention kernel serves these sizes, and the most tokens one entry of its ``tiles`` may hold:
    ``("mma", 32 // group)`` for a bf16 cache the tensor-core kernel can take (32 query rows per CTA), else
    ``("general", 16 // min(group, 4))`` (fp32 cache, odd head sizes; TL_PAGED_MMA=0 forces it)."""
    lib = library()
    if dtype == torch.bfloat16 and os.environ.get("TL_PAGED_MMA", "1") != "0" and lib.tlb_paged_attention_mma_supported(dk, dv, kv_heads, page_size):
        name, n = "mma", int(lib.tlb_paged_attention_mma_tile_tokens(heads, kv_heads))
    else:
        name, n = "general", int(lib.tlb_paged_attention_tile_tokens(heads, kv_heads))
    if n <= 0:
        raise RuntimeError(f"paged_attention: {heads} heads do not divide into {kv_heads} key/value heads")
    return name, n


def paged_attention_tile_tokens(heads: int, kv_heads: int) -> int:
    """The most tokens an entry of ``tiles`` may hold for the general ``paged_attention`` kernel with these head counts."""
    return paged_attention_kernel(torch.float32, heads, kv_heads, 1, 1, 32)[1]


def kv_prepare(q, k, v, *, q_norm=None, k_norm=None, eps: float = 0.0, tok_pos=None, tok_seq=None, block_table=None, slab=None):
    """``q [T, H, dk]`` (a view; normed in place when ``q_norm`` is given), ``k [T, G, dk]``, ``v [T, G, dv]`` (views, or
    None for a layer that reads another layer's cache): optional per-head RMS norms, then keys and values go to every
    token's slot of ``slab [P, page, G * (dk + dv)]``."""
    _gpu("kv_prepare", q, k, v, q_norm, k_norm, tok_pos, tok_seq, block_table, slab)
    T, H, dk = q.shape
    G = dv = 0
    if k is not None:
        G, dv = k.shape[1], v.shape[2]
        P, page_size, width = slab.shape
        if k.shape != (T, G, dk) or v.shape[:2] != (T, G) or width != G * (dk + dv) or not (q.dtype == k.dtype == v.dtype == slab.dtype):
            raise RuntimeError("kv_prepare: keys, values and cache do not match")
        if k.stride(2) != 1 or v.stride(2) != 1 or not slab.is_contiguous():
            raise RuntimeError("kv_prepare: unit inner strides wanted")
    elif q_norm is None:
        return
    if q.stride(2) != 1:
        raise RuntimeError("kv_prepare: unit inner strides wanted")
    P, page_size = (slab.shape[0], slab.shape[1]) if slab is not None else (0, 0)
    _check(library().tlb_kv_prepare(_ptr(q), q.stride(0), q.stride(1), H, _ptr(q_norm), _ptr(k), k.stride(0) if k is not None else 0,
                                    k.stride(1) if k is not None else 0, _ptr(v), v.stride(0) if v is not None else 0, v.stride(1) if v is not None else 0,
                                    G, dk, max(dv, 1), _ptr(k_norm), float(eps), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table),
                                    block_table.shape[1] if block_table is not None else 0, P, page_size, _ptr(slab), T, _code(q.dtype), _stream(q)))


def qk_whole_prepare(q, k, v, *, heads: int, kv_heads: int, q_norm=None, k_norm=None, eps: float = 0.0, rot_dims: int = 0, base: float = 10000.0,
                     interleaved: bool = False, tok_pos, tok_seq=None, block_table=None, slab=None, rope=None):
    """``q [T, heads * dk]`` (a view, changed in place), ``k [T, kv_heads * dk]``, ``v [T, kv_heads * dv]`` (views, or None for
    queries only): RMS norms over the WHOLE projection (weights of that size), rotation of the first ``rot_dims`` entries of
    every head by the token's position, keys and values stored at the token's slot of ``slab [P, page, kv_heads * (dk + dv)]``.
    ``rope`` = (cos, sin) of ``rope_table`` for this step's tokens: the angles are read instead of evaluated."""
    _gpu("qk_whole_prepare", q, k, v, q_norm, k_norm, tok_pos, tok_seq, block_table, slab)
    T = q.shape[0]
    dk = q.shape[1] // heads
    dv = 0
    if q.stride(1) != 1 or q.shape[1] != heads * dk or (q_norm is not None and (q_norm.shape != (heads * dk,) or q_norm.dtype != q.dtype)):
        raise RuntimeError("qk_whole_prepare: queries [T, heads * dk] with unit inner stride, a norm weight of that width")
    cs = sn = None
    if rope is not None and rot_dims:
        cs, sn = rope
        if cs.shape != (T, rot_dims // 2) or sn.shape != cs.shape or cs.dtype != torch.float32 or not cs.is_contiguous() or not sn.is_contiguous():
            raise RuntimeError("qk_whole_prepare: rotation tables must be float32 [T, rot_dims / 2]")
    P = page_size = 0
    if k is not None:
        dv = v.shape[1] // kv_heads
        P, page_size, width = slab.shape
        if k.shape != (T, kv_heads * dk) or v.shape != (T, kv_heads * dv) or width != kv_heads * (dk + dv) or not (q.dtype == k.dtype == v.dtype == slab.dtype):
            raise RuntimeError("qk_whole_prepare: keys, values and cache do not match")
        if k.stride(1) != 1 or v.stride(1) != 1 or not slab.is_contiguous() or (k_norm is not None and (k_norm.shape != (kv_heads * dk,) or k_norm.dtype != q.dtype)):
            raise RuntimeError("qk_whole_prepare: unit inner strides, a norm weight of the keys' width")
    _check(library().tlb_qk_whole_prepare(_ptr(q), q.stride(0), heads, _ptr(q_norm), _ptr(k), k.stride(0) if k is not None else 0, _ptr(v),
                                          v.stride(0) if v is not None else 0, kv_heads if k is not None else 0, dk, max(dv, 1), _ptr(k_norm), float(eps),
                                          int(rot_dims), int(bool(interleaved)), float(base), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table),
                                          block_table.shape[1] if block_table is not None else 0, P, page_size, _ptr(slab), _ptr(cs), _ptr(sn), T, _code(q.dtype),
                                          _stream(q)))


def paged_attention(q, slab, block_table, tiles, tok_pos, *, kv_heads: int, dv: int, mask: int, mask_size: int, scale: float, softcap: float = 0.0,
                    sink: bool = False, gate=None, out=None, kernel: str = "general", max_context: int = 0, head_bias=None, weights: int = 0):
    """``q [T, H, dk]`` (a view with unit inner stride) against ``slab [P, page, kv_heads * (dk + dv)]`` -> ``out [T, H, dv]``
    (contiguous, the query's dtype).  ``gate [T, H]`` (a view with unit inner stride): logits of a sigmoid output gate.
    ``kernel`` and the tile size of ``tiles`` come from ``paged_attention_kernel``.  ``max_context`` (the longest sequence of
    the step, 0 = unknown) lets the tensor-core kernel split the key range over several CTAs when the launch alone would
    leave SMs idle.  ``head_bias`` (fp32 ``[H]``): with ``sink`` the sink's term is ``exp(head_bias[h])`` instead of ``exp(0)``;
    with ``weights=WEIGHTS_SIGMOID`` there is no softmax, a visible key weighs ``sigmoid(score + head_bias[h])``."""
    _gpu("paged_attention", q, slab, block_table, tiles, tok_pos, gate, out, head_bias)
    if head_bias is not None and (head_bias.dtype != torch.float32 or head_bias.shape != (q.shape[1],) or not head_bias.is_contiguous()):
        raise RuntimeError("paged_attention: head_bias must be float32 [H]")
    _contig("paged_attention", slab, block_table, tiles, tok_pos)
    T, H, dk = q.shape
    P, page_size, width = slab.shape
    if width != kv_heads * (dk + dv) or q.dtype != slab.dtype or q.stride(2) != 1:
        raise RuntimeError("paged_attention: query and cache do not match")
    if gate is not None and (gate.shape != (T, H) or gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise RuntimeError("paged_attention: gate must be [T, H] of the query's dtype")
    if out is None:
        out = torch.empty((T, H, dv), dtype=q.dtype, device=q.device)
    if kernel == "mma":
        if slab.dtype != torch.bfloat16:
            raise RuntimeError("paged_attention: the tensor-core kernel takes a bfloat16 cache")
        lib = library()
        reach = min(max_context, int(mask_size)) if mask != MASK_CAUSAL else max_context  # keys a query can see at most
        group = H // kv_heads
        ctas = tiles.shape[0] * kv_heads * -(-group // min(group, 32))
        splits = attention_splits(ctas, reach, slab.device) if reach else 1
        nbytes = int(lib.tlb_paged_attention_mma_workspace(tiles.shape[0], H, kv_heads, dv, splits))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=slab.device) if nbytes else None
        _check(lib.tlb_paged_attention_mma(_ptr(q), q.stride(0), q.stride(1), _ptr(slab), P, page_size, dk, dv, H, kv_heads, _ptr(block_table),
                                           block_table.shape[1], _ptr(tiles), tiles.shape[0], _ptr(tok_pos), int(mask), int(mask_size),
                                           float(scale), float(softcap or 0.0), int(bool(sink)), _ptr(gate),
                                           gate.stride(0) if gate is not None else 0, _ptr(out), out.stride(0), out.stride(1), splits, _ptr(ws), nbytes,
                                           _ptr(head_bias), int(weights), _stream(q)))
        return out
    if kernel != "general":
        raise RuntimeError(f"paged_attention: unknown kernel {kernel!r}")
    _check(library().tlb_paged_attention(_ptr(q), q.stride(0), q.stride(1), _ptr(slab), P, page_size, dk, dv, H, kv_heads, _ptr(block_table),
                                         block_table.shape[1], _ptr(tiles), tiles.shape[0], _ptr(tok_pos), int(mask), int(mask_size), float(scale),
                                         float(softcap or 0.0), int(bool(sink)), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out),
                                         out.stride(0), out.stride(1), _ptr(head_bias), int(weights), _code(q.dtype), _stream(q)))
    return out


def decay_scan(q, k, v, z, z_bias, *, tau: float = 1.0, q_scale: float, seq_info, state, out=None, max_tokens: int | None = None, head_decay=None,
               rope=None, rope_dims: int = 0, rope_interleaved: bool = False, decay_kind: int = 0, a_log=None, bonus=None, skip=None):
    """Linear attention with per-channel decay ``sigmoid(z + z_bias)^(1/tau)``: ``q, k [T, H, dk]``, ``v [T, H, dv]`` views,
    ``z [T, H * dk]`` fp32, ``seq_info [S, 4]`` int32 (first token, count, start position, slot), ``state [slots, H, dk, dv]``
    fp32 (a view whose slots may be further apart) -> fp32 ``[T, H, dv]``.  ``max_tokens``: the largest count in
    ``seq_info`` (default: all tokens); portions longer than a segment run as parallel segments over a workspace.
    ``head_decay`` (fp32 ``[H]``) replaces the logits by one fixed decay per head (``z`` None).  ``rope`` = (cos, sin) tables
    of ``rope_table`` for this step's tokens: the first ``rope_dims`` entries of every head of q and k are rotated in fp32
    on their way in.  ``decay_kind``: ``DECAY_SIGMOID`` as above; ``DECAY_DOUBLE_EXP`` = ``exp(-exp(z + z_bias))`` per key channel;
    ``DECAY_STEP`` = one decay per head and token, ``exp(-exp(a_log[h]) dt)`` with ``dt = softplus(z[t, h] + z_bias[h])``
    (``z [T, H]``), the key multiplied by ``dt``.  ``q, k`` may have fewer heads than ``v`` (``[T, G, dk]``, head h reads
    ``h // (H // G)``).  ``skip [H]``: ``out += skip[h] v``.  ``bonus [H, dk]``: the read-out comes before the update and
    weighs the token's own ``k v^T`` by it."""
    _gpu("decay_scan", q, k, v, z, z_bias, seq_info, state, out, head_decay, a_log, bonus, skip)
    T, G, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    if k.shape != (T, G, dk) or v.shape[0] != T or H % G:
        raise RuntimeError("decay_scan: shapes do not match")
    for name, t, shape in (("a_log", a_log, (H,)), ("bonus", bonus, (H, dk)), ("skip", skip, (H,))):
        if t is not None and (t.shape != shape or t.dtype != q.dtype or not t.is_contiguous()):
            raise RuntimeError(f"decay_scan: {name} must be {shape} of the activations' dtype")
    if decay_kind == DECAY_STEP:
        if z is None or z.shape != (T, H) or z.dtype != torch.float32 or z.stride(1) != 1 or a_log is None or head_decay is not None:
            raise RuntimeError("decay_scan: a step decay takes z [T, H] float32 and a_log [H]")
    elif head_decay is not None:
        if z is not None or head_decay.dtype != torch.float32 or head_decay.shape != (H,) or not head_decay.is_contiguous():
            raise RuntimeError("decay_scan: head_decay must be float32 [H] and replaces z")
    elif z is None or z.shape != (T, H * dk) or z.dtype != torch.float32 or z.stride(1) != 1:
        raise RuntimeError("decay_scan: shapes do not match")
    if z_bias is not None and (z_bias.dtype != q.dtype or not z_bias.is_contiguous()):
        raise RuntimeError("decay_scan: z_bias must be contiguous in the activations' dtype")
    cs = sn = None
    if rope_dims:
        cs, sn = rope
        if cs.shape != (T, rope_dims // 2) or sn.shape != cs.shape or cs.dtype != torch.float32 or not cs.is_contiguous() or not sn.is_contiguous() or rope_dims > dk:
            raise RuntimeError("decay_scan: rotation tables must be float32 [T, rope_dims / 2]")
    if q.stride(2) != 1 or k.stride(2) != 1 or v.stride(2) != 1 or not (q.dtype == k.dtype == v.dtype):
        raise RuntimeError("decay_scan: unit inner strides and one dtype wanted")
    if state.dtype != torch.float32 or state.shape[1:] != (H, dk, dv) or not state[0].is_contiguous():
        raise RuntimeError("decay_scan: state must be float32 [slots, H, dk, dv]")
    if seq_info.dtype != torch.int32 or seq_info.dim() != 2 or seq_info.shape[1] != 4 or not seq_info.is_contiguous():
        raise RuntimeError("decay_scan: seq_info must be int32 [S, 4]")
    if out is None:
        out = torch.empty((T, H, dv), dtype=torch.float32, device=q.device)
    longest = T if max_tokens is None else max(1, min(int(max_tokens), T))
    lib = library()
    nbytes = int(lib.tlb_decay_scan_workspace(seq_info.shape[0], longest, H, dk, dv))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device) if nbytes else None
    _check(lib.tlb_decay_scan(_ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1), _ptr(v), v.stride(0), v.stride(1), _ptr(z),
                              z.stride(0) if z is not None else 0, _ptr(z_bias), float(tau), _ptr(head_decay), _ptr(cs), _ptr(sn), int(rope_dims),
                              int(bool(rope_interleaved)), float(q_scale), H, dk, dv, _ptr(seq_info), seq_info.shape[0], longest, _ptr(state),
                              state.stride(0), state.shape[0], _ptr(out), _ptr(ws), nbytes, int(decay_kind), _ptr(a_log), _ptr(bonus), G, _ptr(skip),
                              _code(q.dtype), _stream(q)))
    return out


def head_norm_gate(o, weight, eps: float, gate=None, act: int = 1, gate_first: bool = False):
    """``o [T, H, dv]`` fp32 -> ``[T, H * dv]`` in the weight's (without one: the gate's) dtype: per-head RMS norm times
    ``weight [dv]`` (None = no weight) times ``silu(gate)`` (``act`` 1), ``sigmoid(gate)`` (2) or ``gate`` (0);
    ``gate [T, H * dv]`` a view with unit inner stride.  A weight of ``[H * dv]`` gives every head its own part;
    ``gate_first``: the gate multiplies ``o`` BEFORE the norm."""
    _gpu("head_norm_gate", o, weight, gate)
    _contig("head_norm_gate", o, weight)
    T, H, dv = o.shape
    if weight is None and gate is None:
        raise RuntimeError("head_norm_gate: a weight or a gate must name the output dtype")
    dtype = weight.dtype if weight is not None else gate.dtype
    wide = weight is not None and weight.shape == (H * dv,) and H > 1
    if o.dtype != torch.float32 or (weight is not None and weight.shape not in ((dv,), (H * dv,))) or (gate is not None and (gate.shape != (T, H * dv) or gate.stride(1) != 1 or gate.dtype != dtype)):
        raise RuntimeError("head_norm_gate: shapes do not match")
    out = torch.empty((T, H * dv), dtype=dtype, device=o.device)
    _check(library().tlb_head_norm_gate(_ptr(o), _ptr(weight), float(eps), _ptr(gate), gate.stride(0) if gate is not None else 0, int(act), _ptr(out),
                                        T, H, dv, int(wide), int(bool(gate_first)), _code(dtype), _stream(o)))
    return out


def delta_scan(q, k, v, beta, a, a_log, dt_bias, *, per_channel: bool, q_scale: float, unit_eps: float = 1e-6, seq_info, state, out=None,
               max_tokens: int | None = None):
    """Gated delta rule: ``q, k [T, G, dk]``, ``v [T, H, dv]``, ``beta [T, H]`` (logits) views in one dtype; ``a`` the decay
    input, ``[T, H]`` (one decay per head, ``dt_bias [H]``) or ``[T, H * dk]`` (one per key channel, ``dt_bias [H * dk]``),
    fp32 or that dtype; ``a_log [H]``; ``state [slots, H, dk, dv]`` fp32 -> fp32 ``[T, H, dv]``.  ``max_tokens``: the largest
    count in ``seq_info`` (default: all tokens); portions longer than a segment run as parallel segments over a workspace."""
    _gpu("delta_scan", q, k, v, beta, a, a_log, dt_bias, seq_info, state, out)
    _contig("delta_scan", a_log, dt_bias, seq_info)
    T, G, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    if k.shape != (T, G, dk) or v.shape[0] != T or beta.shape != (T, H) or H % G or a_log.shape != (H,):
        raise RuntimeError("delta_scan: shapes do not match")
    if a.shape != ((T, H * dk) if per_channel else (T, H)) or dt_bias.numel() != (H * dk if per_channel else H):
        raise RuntimeError("delta_scan: the decay input must be [T, H] or [T, H * dk] with a bias of that width")
    if q.stride(2) != 1 or k.stride(2) != 1 or v.stride(2) != 1 or beta.stride(1) != 1 or a.stride(1) != 1 or not (q.dtype == k.dtype == v.dtype == beta.dtype == a_log.dtype == dt_bias.dtype):
        raise RuntimeError("delta_scan: unit inner strides and one dtype wanted")
    if a.dtype not in (torch.float32, q.dtype):
        raise RuntimeError("delta_scan: the decay input must be float32 or the activations' dtype")
    if state.dtype != torch.float32 or state.shape[1:] != (H, dk, dv) or not state[0].is_contiguous():
        raise RuntimeError("delta_scan: state must be float32 [slots, H, dk, dv]")
    if seq_info.dtype != torch.int32 or seq_info.dim() != 2 or seq_info.shape[1] != 4:
        raise RuntimeError("delta_scan: seq_info must be int32 [S, 4]")
    if out is None:
        out = torch.empty((T, H, dv), dtype=torch.float32, device=q.device)
    longest = T if max_tokens is None else max(1, min(int(max_tokens), T))
    lib = library()
    nbytes = int(lib.tlb_delta_scan_workspace(seq_info.shape[0], longest, H, dk, dv))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device) if nbytes else None
    _check(lib.tlb_delta_scan(_ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1), _ptr(v), v.stride(0), v.stride(1), _ptr(beta),
                              beta.stride(0), _ptr(a), int(a.dtype == torch.float32), a.stride(0), int(per_channel), _ptr(a_log), _ptr(dt_bias),
                              float(q_scale), float(unit_eps), H, G, dk, dv, _ptr(seq_info), seq_info.shape[0], longest, _ptr(state), state.stride(0),
                              state.shape[0], _ptr(out), _ptr(ws), nbytes, _code(q.dtype), _stream(q)))
    return out


def short_conv(x, taps, *, seq_info, state, max_tokens: int, act: int = 1, bias=None, add_input: bool = False):
    """Causal convolution per channel along every sequence (plus ``bias [C]``; plus the input itself, ``add_input``), then silu
    (``act`` 1) or nothing (0): ``x [T, C]`` (a view with unit inner
    stride), ``taps [C, K]``, ``state [slots, C, K - 1]`` fp32 (a view whose slots may be further apart): the inputs before
    the step's first token, replaced by the step's last ones -> ``[T, C]`` contiguous in x's dtype."""
    _gpu("short_conv", x, taps, seq_info, state, bias)
    _contig("short_conv", taps, seq_info, bias)
    if bias is not None and (bias.shape != (x.shape[1],) or bias.dtype != x.dtype):
        raise RuntimeError("short_conv: bias must be [C] of x's dtype")
    T, C = x.shape
    K = taps.shape[1]
    if taps.shape[0] != C or taps.dtype != x.dtype or x.stride(1) != 1:
        raise RuntimeError("short_conv: taps must be [C, K] of x's dtype")
    if K > 1 and (state is None or state.dtype != torch.float32 or state.shape[1:] != (C, K - 1) or not state[0].is_contiguous()):
        raise RuntimeError("short_conv: state must be float32 [slots, C, K - 1]")
    y = torch.empty((T, C), dtype=x.dtype, device=x.device)
    _check(library().tlb_short_conv(_ptr(x), x.stride(0), _ptr(taps), _ptr(bias), int(bool(add_input)), C, K, int(act), _ptr(seq_info), seq_info.shape[0], max(1, int(max_tokens)),
                                    _ptr(state) if K > 1 else None, state.stride(0) if K > 1 else 0, state.shape[0] if K > 1 else 0, _ptr(y),
                                    _code(x.dtype), _stream(x)))
    return y


def act_rows(x: torch.Tensor, act: int) -> torch.Tensor:
    """``act(x)`` elementwise (``ACT_SILU``, ``ACT_GELU_TANH``, ``ACT_RELU_SQUARED``, ``ACT_TANH``)."""
    _gpu("act_rows", x)
    _contig("act_rows", x)
    out = torch.empty_like(x)
    _check(library().tlb_act_rows(_ptr(x), _ptr(out), x.shape[0], x.shape[1], int(act), _code(x.dtype), _stream(x)))
    return out


def softcap_rows(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``cap * tanh(x / cap)`` of fp32 ``[rows, width]``, in place."""
    _gpu("softcap_rows", x)
    _contig("softcap_rows", x)
    if x.dtype != torch.float32 or x.dim() != 2:
        raise RuntimeError("softcap_rows: expected float32 [rows, width]")
    _check(library().tlb_softcap_rows(_ptr(x), x.shape[0], x.shape[1], float(cap), _stream(x)))
    return x


def cast_rows(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """``dst[:, :] = src`` rounded to dst's dtype; ``src`` fp32 ``[rows, dim]`` contiguous, ``dst`` a column block (unit
    inner stride) of a wider matrix."""
    _gpu("cast_rows", src, dst)
    _contig("cast_rows", src)
    if src.dtype != torch.float32 or src.shape != dst.shape or dst.stride(1) != 1:
        raise RuntimeError("cast_rows: float32 [rows, dim] into a view of the same shape")
    _check(library().tlb_cast_rows(_ptr(src), _ptr(dst), dst.stride(0), src.shape[0], src.shape[1], _code(dst.dtype), _stream(src)))
    return dst


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    _gpu("argmax_rows", logits)
    _contig("argmax_rows", logits)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise RuntimeError("argmax_rows: expected float32 [rows, vocab]")
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _check(library().tlb_argmax_rows(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], _stream(logits)))
    return out


def streams_step(xs, *, x0=None, y=None, y_bias=None, write=None, read=None, eps: float = 0.0, dtype=None):
    """Residual streams ``xs [rows, n, dim]`` fp32 (in place) around a sublayer.  ``write`` (fp32 ``[n * n + n]``: the mixing
    matrix indexed [from, to], then the output weights) with the sublayer's output ``y [rows, dim]`` fp32 (+ ``y_bias [dim]``):
    ``x_t <- sum_s mix[s, t] x_s + out[t] (y + y_bias)``.  ``read`` (fp32 ``[n + 1]``: the input weights, then the norm's one
    weight): returns ``rms_norm(sum_s in[s] x_s) * g`` rounded to ``dtype``.  ``x0 [rows, dim]`` fp32: every stream starts as
    that row."""
    _gpu("streams_step", xs, x0, y, y_bias, write, read)
    _contig("streams_step", xs, x0, y, y_bias, write, read)
    rows, n, dim = xs.shape
    if xs.dtype != torch.float32 or any(t is not None and (t.dtype != torch.float32 or t.shape != (rows, dim)) for t in (x0, y)):
        raise RuntimeError("streams_step: streams [rows, n, dim], x0 and y [rows, dim] must be float32")
    if (write is not None and (y is None or write.dtype != torch.float32 or write.numel() != n * n + n)) or (read is not None and (read.dtype != torch.float32 or read.numel() != n + 1)):
        raise RuntimeError("streams_step: write must be float32 [n * n + n] (with y), read float32 [n + 1]")
    if y_bias is not None:
        dtype = y_bias.dtype
    h = None
    if read is not None:
        if dtype is None:
            raise RuntimeError("streams_step: name the dtype of the norm's output")
        h = torch.empty((rows, dim), dtype=dtype, device=xs.device)
    _check(library().tlb_streams_step(_ptr(xs), _ptr(x0), _ptr(y), _ptr(y_bias), _ptr(write), _ptr(read), float(eps), _ptr(h), rows, n, dim,
                                      _code(dtype if dtype is not None else torch.float32), _stream(xs)))
    return h


def shift_mix(h, mu, *, seq_info, state, max_tokens: int):
    """Token shift: ``out[i, t] = h[t] + (h[t-1] - h[t]) * mu[i]`` along every sequence; ``h [T, dim]`` (unit inner stride),
    ``mu [n, dim]`` (n <= 8), ``state [slots, dim]`` fp32 (a view whose slots may be further apart): the row before the step's
    first token, replaced by the step's last one; zero before position 0 -> ``[n, T, dim]``."""
    _gpu("shift_mix", h, mu, seq_info, state)
    _contig("shift_mix", mu, seq_info)
    T, dim = h.shape
    n = mu.shape[0]
    if mu.shape != (n, dim) or mu.dtype != h.dtype or h.stride(1) != 1 or n > 8:
        raise RuntimeError("shift_mix: mu must be [n <= 8, dim] of h's dtype")
    if state.dtype != torch.float32 or state.shape[1:] != (dim,) or state.stride(1) != 1:
        raise RuntimeError("shift_mix: state must be float32 [slots, dim]")
    out = torch.empty((n, T, dim), dtype=h.dtype, device=h.device)
    _check(library().tlb_shift_mix(_ptr(h), h.stride(0), _ptr(mu), n, dim, _ptr(seq_info), seq_info.shape[0], max(1, int(max_tokens)), _ptr(state),
                                   state.stride(0), state.shape[0], _ptr(out), T * dim, _code(h.dtype), _stream(h)))
    return out
