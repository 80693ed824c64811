"""Python face of the CUDA kernels: argument checks, then one C call per op.

Every function takes device tensors, writes into caller-provided outputs, launches on the
current CUDA stream and allocates nothing.  A tensor that is not on a CUDA device, has the
wrong dtype or is not contiguous raises :class:`KernelError` before anything is launched;
the native side checks sizes again and reports through ``ftk_last_error``.

Kernel inventory (reference kernel each one stands for):

=====================  ==========================================================
embedding_gather       python/freetoken/kernel/csrc/jit/index.cu:31-59
add_rmsnorm            python/freetoken/kernel/triton/norm.py:42-112
norm_rope_store        norm.py:42-75 + python/freetoken/kernel/triton/rope.py:28-91 +
                       python/freetoken/kernel/csrc/jit/store.cu:27-53, in one pass
paged_attention        python/freetoken/kernel/triton/attention.py:147-466,469-880
router_topk            python/freetoken/models/minimax_m3/moe.py:71-81
moe_permute            python/freetoken/kernel/triton/fused_moe.py:5-108
moe_gemm1_act          fused_moe.py:156-302 + python/freetoken/kernel/triton/activation.py:67-112
moe_gemm2              fused_moe.py:156-302 (route weight on the accumulator, :292-296)
moe_combine            fused_moe.py:111-153
act_and_mul            activation.py:67-112
sample                 python/freetoken/engine/sample.py:24-80, python/freetoken/kernel/triton/sampling.py
moe_route              router product + router_topk + moe_permute in one launch (short steps)
add_rmsnorm_routes     moe_combine + add_rmsnorm in one pass
linear                 python/freetoken/layers/linear.py:66-70 (the library product)
copy_tokens            the sampled tokens of the step before, taken on the device
                       (python/freetoken/scheduler/scheduler.py:194-256, overlapped scheduling)
=====================  ==========================================================

``paged_attention`` runs one of five kernels by ``tile_rows``: 16 (float32, or bfloat16 steps of single
tokens where the tcgen05 kernel does not take the sizes), 64 (bfloat16 mma.sync), 128 (bfloat16 tcgen05:
long steps and decode steps), 256 (the same with two query tiles per CTA: very long steps).
"""

from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from ..errors import KernelError
from . import library

F32, BF16 = 0, 1
ACT_SILU, ACT_SWIGLUOAI = 0, 1
SCORE_SIGMOID, SCORE_SOFTMAX = 0, 1
ACT_CODES = {"silu": ACT_SILU, "swigluoai": ACT_SWIGLUOAI}
SCORE_CODES = {"sigmoid": SCORE_SIGMOID, "softmax": SCORE_SOFTMAX}

_vp = ctypes.c_void_p
_i = ctypes.c_int
_f = ctypes.c_float


class _Section(ctypes.Structure):
    _fields_ = [
        ("first_head", _i), ("n_heads", _i), ("norm_weight", _vp), ("rotate", _i),
        ("dense_out", _vp), ("slab", _vp), ("slot_map", _vp), ("page_size", _i), ("num_pages", _i),
    ]


_SIGNATURES = {
    "ftk_embedding_gather": [_vp, _i, _vp, _i, _i, _i, _vp, _vp],
    "ftk_add_rmsnorm": [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _i, _vp],
    "ftk_add_rmsnorm_routes": [_vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _i, _vp],
    "ftk_norm_rope_store": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _i, _i,
                            ctypes.POINTER(_Section), _vp],
    "ftk_paged_attention": [_vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                            _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ftk_attention_tc_fits": [_i, _i, _i],
    "ftk_paged_attention_tc": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                               _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ftk_attention_tc_few_fits": [_i, _i, _i],
    "ftk_paged_attention_tc_few": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                                      _i, _i, _i, _i, _i, _i, ctypes.c_float, _i, _vp],
    "ftk_paged_attention_tc_pair": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                                    _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ftk_paged_attention_sparse": [_vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                                   _i, _i, _i, _i, _i, _i, _f, _vp, _i, _i, _vp],
    "ftk_sparse_select": [_vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp],
    "ftk_sparse_score_fits": [_i, _i, _i],
    "ftk_router_topk": [_vp, _i, _vp, _i, _i, _i, _i, _f, _vp, _vp, _vp],
    "ftk_moe_permute": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "ftk_moe_route_fits": [_i, _i, _i, _i],
    "ftk_moe_route": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp],
    "ftk_small_linear_fits": [_i, _i, _i],
    "ftk_small_linear": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "ftk_moe_small_fits": [_i, _i, _i, _i],
    "ftk_moe_small_gate_up": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp],
    "ftk_moe_small_down": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ftk_moe_gather": [_vp, _i, _vp, _i, _i, _i, _vp, _vp],
    "ftk_moe_gemm1_act": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "ftk_moe_gemm1_gather_fits": [_i, _i, _i, _i],
    "ftk_moe_gemm1_act_gather": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "ftk_moe_gemm2": [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ftk_moe_combine": [_vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp],
    "ftk_act_and_mul": [_vp, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "ftk_sample": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "ftk_cast": [_vp, _i, _vp, _i, ctypes.c_longlong, _vp],
    "ftk_table_update": [_vp, ctypes.c_longlong, _vp, _i, _vp],
    "ftk_copy_tokens": [_vp, _i, _vp, _vp, _i, _i, _i, _vp],
    "ftk_read_status": [ctypes.POINTER(ctypes.c_int)],
    "ftk_set_moe_tensor_cores": [_i],
    "ftk_set_moe_pairs": [_i],
    "ftk_debug_set_status": [_i, _i],
    "ftk_variant_counts": [ctypes.c_char_p, _i, _i],
}
_bound = False
_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (graph replays add their recorded count)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _lib():
    global _bound
    lib = library.load()
    if not _bound:
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i
        _bound = True
    return lib


def _check(status: int, name: str, launches: int = 1) -> None:
    global _launches
    _launches += launches
    if status != 0:
        msg = library.load().ftk_last_error()
        raise KernelError(f"{name}: {msg.decode() if msg else 'error ' + str(status)}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor, what: str) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)")


def _dev(t: Optional[torch.Tensor], what: str, dtype: Optional[torch.dtype] = None) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on '{t.device}', the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    return t.data_ptr()


def read_status() -> int:
    """Code left by a kernel whose bounded wait ran out since the last call (0 = none).  Waits
    for the device.  101-104 come from the tensor-core grouped GEMM (producer, accumulator
    hand-back, operand arrival, accumulator arrival)."""
    out = (ctypes.c_int * 2)()
    status = _lib().ftk_read_status(out)
    if status != 0:
        raise KernelError("read_status: " + library.load().ftk_last_error().decode())
    return int(out[0])


def check_status() -> None:
    code = read_status()
    if code:
        raise KernelError(f"a kernel gave up waiting (status {code}); its results are not valid")


def variant_counts(reset: bool = False) -> dict:
    """Launches so far by the form of kernel they took (``"attention: tcgen05, 128-row query tiles"``,
    ``"expert gate/up product: tcgen05, 64 tokens a tile, deep pipeline"``, ``"route sort: three passes over
    128-route segments"`` ...): what a step really ran, for tests and measurements.  Launches replayed from
    a CUDA graph were counted when the graph was recorded."""
    lib = _lib()
    need = lib.ftk_variant_counts(None, 0, 0)
    buf = ctypes.create_string_buffer(need + 256)
    lib.ftk_variant_counts(buf, len(buf), 1 if reset else 0)
    out = {}
    for line in buf.value.decode().splitlines():
        name, _, n = line.rpartition("\t")
        out[name] = int(n)
    return out


def debug_set_status(unit: int, code: int) -> None:
    """Write ``code`` into a status word from the host (``unit`` 0: grouped GEMM, 1: attention), as a
    kernel whose bounded wait ran out would have.  For tests of the error path; nothing waits."""
    _check(_lib().ftk_debug_set_status(int(unit), int(code)), "debug_set_status", 0)


def set_moe_tensor_cores(enabled: bool) -> None:
    """False sends bfloat16 grouped expert products to the CUDA-core kernels (comparisons only)."""
    _lib().ftk_set_moe_tensor_cores(1 if enabled else 0)


def set_moe_pairs(enabled: bool) -> None:
    """False keeps expert products with 128- and 256-token tiles on the one-CTA form of the tcgen05 kernel instead
    of pairs of CTAs (comparisons only)."""
    _lib().ftk_set_moe_pairs(1 if enabled else 0)


# --------------------------------------------------------------------------- elementwise
def embedding_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, :] = float32(table[ids[t], :])``; ``out`` is the 32-bit residual stream."""
    V, H = table.shape
    T = ids.shape[0]
    if out.shape != (T, H):
        raise KernelError(f"embedding_gather: out shape {tuple(out.shape)} != {(T, H)}")
    _check(_lib().ftk_embedding_gather(_dev(table, "table"), _code(table, "table"),
                                       _dev(ids, "ids", torch.int32), T, H, V,
                                       _dev(out, "out", torch.float32), _stream()),
           "embedding_gather")


def add_rmsnorm(x: Optional[torch.Tensor], residual: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, gemma: bool, out: torch.Tensor, out_f32: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> None:
    """RMSNorm with the residual sum fused in.

    ``z = x + residual`` in 32-bit (either may be None); without ``rows`` the sum is stored
    back to ``residual``; ``out = z * rsqrt(mean(z^2) + eps) * (1 + w)`` (``w`` when not
    ``gemma``).  With ``rows`` only those rows are read and ``out[i]`` belongs to
    ``rows[i]``; the residual stays as it is.  ``out_f32`` receives ``float32(out)``.
    """
    src = x if x is not None else residual
    if src is None:
        raise KernelError("add_rmsnorm: x and residual are both None")
    H = src.shape[-1]
    n_rows = rows.shape[0] if rows is not None else src.numel() // H
    if weight.shape != (H,):
        raise KernelError(f"add_rmsnorm: weight shape {tuple(weight.shape)} != {(H,)}")
    if out.numel() != n_rows * H:
        raise KernelError(f"add_rmsnorm: out has {out.numel()} elements, expected {n_rows * H}")
    if out_f32 is not None and out_f32.numel() != n_rows * H:
        raise KernelError("add_rmsnorm: out_f32 has the wrong size")
    _check(_lib().ftk_add_rmsnorm(_dev(x, "x"), _code(x, "x") if x is not None else F32,
                                  _dev(residual, "residual", torch.float32),
                                  _dev(weight, "weight", torch.float32),
                                  _dev(out, "out"), _code(out, "out"),
                                  _dev(out_f32, "out_f32", torch.float32),
                                  _dev(rows, "rows", torch.int32), n_rows, H, float(eps),
                                  1 if gemma else 0, _stream()), "add_rmsnorm")


def add_rmsnorm_routes(y: torch.Tensor, route_pos: torch.Tensor, top_k: int, shared: Optional[torch.Tensor],
                       residual: torch.Tensor, weight: torch.Tensor, eps: float, gemma: bool, out: torch.Tensor,
                       out_f32: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """:func:`moe_combine` and :func:`add_rmsnorm` in one pass: the row added to ``residual[t]`` is
    ``sum_j y[route_pos[t*k + j]] (+ shared[t])``, a 32-bit sum in route order rounded to ``y``'s type."""
    R, H = y.shape
    T = residual.numel() // H
    n_rows = rows.shape[0] if rows is not None else T
    if route_pos.numel() != T * top_k or weight.shape != (H,) or out.numel() != n_rows * H:
        raise KernelError("add_rmsnorm_routes: shapes do not agree")
    if shared is not None and (shared.shape != (T, H) or shared.dtype != y.dtype):
        raise KernelError("add_rmsnorm_routes: shared must be [tokens, hidden] of y's dtype")
    if out_f32 is not None and out_f32.numel() != n_rows * H:
        raise KernelError("add_rmsnorm_routes: out_f32 has the wrong size")
    _check(_lib().ftk_add_rmsnorm_routes(_dev(y, "y"), _code(y, "y"), _dev(route_pos, "route_pos", torch.int32), top_k, R,
                                         _dev(shared, "shared"), _dev(residual, "residual", torch.float32),
                                         _dev(weight, "weight", torch.float32), _dev(out, "out"), _code(out, "out"),
                                         _dev(out_f32, "out_f32", torch.float32), _dev(rows, "rows", torch.int32),
                                         n_rows, H, float(eps), 1 if gemma else 0, _stream()), "add_rmsnorm_routes")


def act_and_mul(gate_up: torch.Tensor, out: torch.Tensor, act: str, alpha: float, limit: float) -> None:
    """``out = act(gate_up[:, :I], gate_up[:, I:])`` with ``act`` silu or swigluoai."""
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("act_and_mul: out must be [rows, I] of the input's dtype")
    _check(_lib().ftk_act_and_mul(_dev(gate_up, "gate_up"), _code(gate_up, "gate_up"), n, two_i // 2,
                                  ACT_CODES[act], float(alpha), float(limit), _dev(out, "out"),
                                  _stream()), "act_and_mul")


def table_update(table: torch.Tensor, updates: torch.Tensor, n_updates: int) -> None:
    """``table.flat[updates[i, 0]] = updates[i, 1]`` for ``i < n_updates``; negative indices are skipped."""
    if updates.numel() < 2 * n_updates:
        raise KernelError("table_update: updates shorter than n_updates")
    _check(_lib().ftk_table_update(_dev(table, "table", torch.int32), table.numel(),
                                   _dev(updates, "updates", torch.int32), n_updates, _stream()),
           "table_update")


def copy_tokens(dst: torch.Tensor, pairs: torch.Tensor, src: torch.Tensor, n: int, vocab: int) -> None:
    """``dst[pairs[i, 0]] = src[pairs[i, 1]]`` for ``i < n`` (negative indices skipped; values outside
    the vocabulary become 0): tokens sampled on the device become the next step's inputs."""
    if pairs.numel() < 2 * n:
        raise KernelError("copy_tokens: pairs shorter than n")
    _check(_lib().ftk_copy_tokens(_dev(dst, "dst", torch.int32), dst.numel(), _dev(pairs, "pairs", torch.int32),
                                  _dev(src, "src", torch.int32), src.numel(), n, vocab, _stream()), "copy_tokens")


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    """``dst = src`` converted between float32 and bfloat16 (round to nearest even)."""
    if src.numel() != dst.numel():
        raise KernelError("cast: sizes differ")
    _check(_lib().ftk_cast(_dev(src, "src"), _code(src, "src"), _dev(dst, "dst"), _code(dst, "dst"),
                           src.numel(), _stream()), "cast")


# --------------------------------------------------------------------------- attention
def norm_rope_store(x: torch.Tensor, head_dim: int, rotary_dim: int, positions: torch.Tensor,
                    rope_table: Optional[torch.Tensor], eps: float, gemma: bool,
                    sections: Sequence[dict]) -> None:
    """Per-head RMSNorm, partial NeoX rotation and scatter of projected heads, in one pass.

    ``x [T, n_heads_total * head_dim]`` is cut into sections of whole heads.  A section is a
    dict: ``first_head``, ``n_heads``, ``norm_weight`` (float32 ``[head_dim]`` or None),
    ``rotate`` (bool), and one destination: ``dense_out [T, n_heads, head_dim]`` or
    ``slab [pages, n_heads, page_size, head_dim]`` with ``slot_map [T]`` (slot = page *
    page_size + offset, negative = skip).  ``rope_table [max_pos, rotary_dim]`` holds
    cos then sin of ``position * inv_freq`` in float32.
    """
    T = x.shape[0]
    n_total = x.shape[1] // head_dim
    arr = (_Section * len(sections))()
    keep = []
    for i, s in enumerate(sections):
        if s["first_head"] + s["n_heads"] > n_total:
            raise KernelError("norm_rope_store: section exceeds the heads of x")
        arr[i].first_head = s["first_head"]
        arr[i].n_heads = s["n_heads"]
        arr[i].norm_weight = _dev(s.get("norm_weight"), "norm_weight", torch.float32)
        arr[i].rotate = 1 if s.get("rotate") else 0
        dense, slab = s.get("dense_out"), s.get("slab")
        if (dense is None) == (slab is None):
            raise KernelError("norm_rope_store: a section needs exactly one of dense_out and slab")
        if dense is not None:
            if dense.dtype != x.dtype or dense.numel() != T * s["n_heads"] * head_dim:
                raise KernelError("norm_rope_store: dense_out has the wrong dtype or size")
            arr[i].dense_out = _dev(dense, "dense_out")
        else:
            if slab.dtype != x.dtype or slab.dim() != 4 or slab.shape[1] != s["n_heads"] \
                    or slab.shape[3] != head_dim:
                raise KernelError("norm_rope_store: slab must be [pages, n_heads, page_size, head_dim]")
            arr[i].slab = _dev(slab, "slab")
            arr[i].slot_map = _dev(s["slot_map"], "slot_map", torch.int32)
            if s["slot_map"].shape[0] < T:
                raise KernelError("norm_rope_store: slot_map shorter than the tokens")
            arr[i].num_pages = slab.shape[0]
            arr[i].page_size = slab.shape[2]
        keep.append(s)
    if rotary_dim:
        if rope_table is None or rope_table.shape[1] != rotary_dim:
            raise KernelError("norm_rope_store: rope_table must be [max_pos, rotary_dim]")
    max_pos = rope_table.shape[0] if rope_table is not None else 0
    _check(_lib().ftk_norm_rope_store(_dev(x, "x"), _code(x, "x"), T, x.shape[1], head_dim, rotary_dim,
                                      _dev(positions, "positions", torch.int32),
                                      _dev(rope_table, "rope_table", torch.float32), max_pos,
                                      float(eps), 1 if gemma else 0, len(sections), arr, _stream()),
           "norm_rope_store")


def paged_attention(q: torch.Tensor, k_slab: torch.Tensor, v_slab: torch.Tensor,
                    block_table: torch.Tensor, seg_info: torch.Tensor, n_segs: int,
                    items: torch.Tensor, n_items: int, part_o: Optional[torch.Tensor],
                    part_ml: Optional[torch.Tensor], out: torch.Tensor, tile_rows: int, scale: float,
                    window: Optional[int], sel: Optional[torch.Tensor] = None, block_size: int = 0,
                    few_rows: bool = False) -> None:
    """Causal softmax attention of the step's queries over the paged keys and values.

    ``q, out [T, Hq, D]``; slabs ``[pages, Hkv, page_size, D]``; ``block_table [rows, width]``
    page ids; ``seg_info [S, 4]`` = q_start, q_len, kv_len, block-table row; ``items [W, 8]``
    from :func:`freetoken_b200.engine.attention_plan.build_plan`; ``part_o [slots, Hkv,
    tile_rows, D]`` and ``part_ml [slots, Hkv, tile_rows, 2]`` float32 scratch for split
    tiles.  Query ``t`` of a segment sits at position ``kv_len - q_len + t`` and reads keys at
    positions ``<=`` its own (and ``>`` its own minus ``window`` when a window is given).

    Block-sparse layers pass ``sel [T, Hkv, topk]`` (chosen key blocks of ``block_size`` positions
    per token and KV head, ascending, -1 padded, from :func:`sparse_select`); a query then reads only
    the keys of its chosen blocks, the work items hold one token each and their key ranges count
    chosen keys.

    ``few_rows`` (with ``tile_rows = 16``, bfloat16) runs the tcgen05 kernel in its form for decode
    steps (one warp takes the softmax of a tile's at most 16 rows); its work list has key pieces that
    are multiples of 128 (``build_plan(..., key_tile=128)``).
    """
    T, Hq, D = q.shape
    pages, Hkv, P, D2 = k_slab.shape
    if D2 != D or v_slab.shape != k_slab.shape or Hq % Hkv:
        raise KernelError("paged_attention: q / slab shapes do not agree")
    if out.shape != q.shape or out.dtype != q.dtype or k_slab.dtype != q.dtype:
        raise KernelError("paged_attention: dtypes or out shape do not agree")
    n_slots = part_o.shape[0] if part_o is not None else 0
    if part_o is not None and (part_o.shape[1:] != (Hkv, tile_rows, D) or part_ml is None
                               or part_ml.shape != (n_slots, Hkv, tile_rows, 2)):
        raise KernelError("paged_attention: scratch shapes do not match tile_rows / heads")
    if few_rows and tile_rows != 16:
        raise KernelError(f"paged_attention: few_rows goes with tiles of 16 rows, got {tile_rows}")
    if tile_rows in (128, 256) or few_rows:
        # bfloat16 steps on the tcgen05 kernels: one query tile per CTA, a pair of them, or tiles of a few rows
        if sel is not None or window or q.dtype != torch.bfloat16:
            raise KernelError("paged_attention: the tcgen05 kernels take bfloat16 without window or block selection")
        fn = (_lib().ftk_paged_attention_tc_few if few_rows else
              _lib().ftk_paged_attention_tc_pair if tile_rows == 256 else _lib().ftk_paged_attention_tc)
        _check(fn(
            _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"),
            _dev(block_table, "block_table", torch.int32), block_table.shape[1],
            _dev(seg_info, "seg_info", torch.int32), n_segs,
            _dev(items, "items", torch.int32), n_items,
            _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
            _dev(out, "out"), T, Hq, Hkv, D, P, pages, float(scale), 0, _stream()),
            "paged_attention (tcgen05)", 2 if n_slots else 1)
        return
    if sel is not None:
        if sel.dim() != 3 or sel.shape[0] < T or sel.shape[1] != Hkv or block_size < 1:
            raise KernelError("paged_attention: sel must be [T, Hkv, topk] with a positive block_size")
        _check(_lib().ftk_paged_attention_sparse(
            _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"), _code(q, "q"),
            _dev(block_table, "block_table", torch.int32), block_table.shape[1],
            _dev(seg_info, "seg_info", torch.int32), n_segs,
            _dev(items, "items", torch.int32), n_items,
            _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
            _dev(out, "out"), Hq, Hkv, D, P, pages, tile_rows, float(scale),
            _dev(sel, "sel", torch.int32), sel.shape[2], int(block_size), _stream()),
            "paged_attention (block-sparse)", 2 if n_slots else 1)
        return
    _check(_lib().ftk_paged_attention(
        _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"), _code(q, "q"),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(seg_info, "seg_info", torch.int32), n_segs,
        _dev(items, "items", torch.int32), n_items,
        _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
        _dev(out, "out"), Hq, Hkv, D, P, pages, tile_rows, float(scale),
        int(window) if window else 0, _stream()), "paged_attention", 2 if n_slots else 1)


def attention_tc_fits(head_dim: int, page_size: int, group: int) -> bool:
    """Whether the tcgen05 attention kernel (tiles of 128 query rows) takes these sizes."""
    return bool(_lib().ftk_attention_tc_fits(head_dim, page_size, group))


def attention_tc_few_fits(head_dim: int, page_size: int, group: int) -> bool:
    """Whether the tcgen05 attention kernel takes these sizes in its form for tiles of at most 16 rows."""
    return bool(_lib().ftk_attention_tc_few_fits(head_dim, page_size, group))


def sparse_score_fits(n_heads: int, dim: int, block_size: int) -> bool:
    """Whether bfloat16 block scores of these sizes are taken on the tensor cores (given a ``scores`` scratch)."""
    return bool(_lib().ftk_sparse_score_fits(n_heads, dim, block_size))


def sparse_select(iq: torch.Tensor, ik_slab: torch.Tensor, block_table: torch.Tensor, seg_info: torch.Tensor,
                  n_segs: int, block_size: int, local_blocks: int, init_blocks: int, max_blocks: int,
                  sel: torch.Tensor, scores: Optional[torch.Tensor] = None, live_blocks: int = 0) -> None:
    """Key blocks each new token of a block-sparse layer attends to.

    ``iq [T, Hi, Di]`` index queries, ``ik_slab [pages, 1, page_size, Di]`` cached index keys.  A
    block's score is the largest ``iq . ik`` over its visible positions; the first ``init_blocks``
    and the newest ``local_blocks`` blocks are always taken; the ``min(topk, visible)`` best go to
    ``sel [T, Hi, topk]`` in ascending order, padded with -1.  ``max_blocks`` bounds the blocks of
    the longest request (sizes the kernel's shared memory).  ``scores [T, Hi, max_blocks]`` float32 scratch lets
    bfloat16 scores be contracted on the tensor cores (:func:`sparse_score_fits`), every key read once per
    tile of tokens; without it a CTA per token and head walks the blocks.  ``live_blocks`` (0 = ``max_blocks``):
    blocks that the longest request of this step can hold, which bounds the launch; a step replayed from a
    CUDA graph must give a bound that holds for every replay."""
    T, Hi, Di = iq.shape
    pages, one, P, Di2 = ik_slab.shape
    if one != 1 or Di2 != Di or ik_slab.dtype != iq.dtype:
        raise KernelError("sparse_select: ik_slab must be [pages, 1, page_size, Di] of iq's dtype")
    if sel.dim() != 3 or sel.shape[0] < T or sel.shape[1] != Hi:
        raise KernelError("sparse_select: sel must be [T, Hi, topk]")
    if scores is not None and (scores.dtype != torch.float32 or scores.numel() < T * Hi * max_blocks):
        raise KernelError("sparse_select: scores must hold [T, Hi, max_blocks] float32")
    _check(_lib().ftk_sparse_select(_dev(iq, "iq"), _dev(ik_slab, "ik_slab"), _code(iq, "iq"),
                                    _dev(block_table, "block_table", torch.int32), block_table.shape[1],
                                    _dev(seg_info, "seg_info", torch.int32), n_segs, T, Hi, Di, P, pages,
                                    int(block_size), sel.shape[2], int(local_blocks), int(init_blocks),
                                    int(max_blocks), int(live_blocks), _dev(sel, "sel", torch.int32),
                                    _dev(scores, "scores", torch.float32), _stream()), "sparse_select",
           2 if scores is not None else 1)


# --------------------------------------------------------------------------- experts
def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, scoring: str,
                scale: float, ids: torch.Tensor, weights: torch.Tensor, n_parts: int = 1) -> None:
    """Expert choice from float32 router logits ``[T, E]``.

    sigmoid: ``s = sigmoid(l)``; choice by ``s + bias``; ``w = s[ids] / (sum + 1e-20) * scale``.
    softmax: ``s = softmax(l)``; choice by ``s (+ bias)``; ``w = s[ids] / sum * scale``.
    The largest goes first; the lower expert index wins a tie.

    With ``n_parts > 1`` the logits come as ``[T, n_parts * E]``: a token's logit of expert ``e`` is the
    32-bit sum of ``logits[t, q * E + e]`` over the parts ``q`` in their order.
    """
    T, PE = logits.shape
    if n_parts < 1 or PE % n_parts or not logits.is_contiguous():
        raise KernelError("router_topk: logits must be contiguous [T, n_parts * E]")
    E = PE // n_parts
    if ids.shape != (T, top_k) or weights.shape != (T, top_k):
        raise KernelError("router_topk: ids / weights must be [T, top_k]")
    if bias is not None and bias.shape != (E,):
        raise KernelError("router_topk: bias must be [E]")
    _check(_lib().ftk_router_topk(_dev(logits, "logits", torch.float32), int(n_parts), _dev(bias, "bias", torch.float32),
                                  T, E, top_k, SCORE_CODES[scoring], float(scale),
                                  _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32),
                                  _stream()), "router_topk")


def moe_permute(topk_ids: torch.Tensor, n_experts: int, expert_counts: torch.Tensor,
                expert_offsets: torch.Tensor, sorted_routes: torch.Tensor, route_pos: torch.Tensor) -> None:
    """Sort the routes ``(t, j)`` by expert, keeping their order within an expert.

    ``expert_counts [E]``: routes per expert;
    ``expert_offsets [E + 1]``: rows of expert ``e`` are ``[offsets[e], offsets[e+1])``;
    ``sorted_routes [T*k]``: route index ``t*k + j`` at each sorted row;
    ``route_pos [T*k]``: sorted row of each route."""
    T, k = topk_ids.shape
    if expert_offsets.shape != (n_experts + 1,) or expert_counts.shape != (n_experts,) \
            or sorted_routes.numel() != T * k \
            or route_pos.numel() != T * k:
        raise KernelError("moe_permute: output shapes are wrong")
    _check(_lib().ftk_moe_permute(_dev(topk_ids, "topk_ids", torch.int32), T, k, n_experts,
                                  _dev(expert_counts, "expert_counts", torch.int32),
                                  _dev(expert_offsets, "expert_offsets", torch.int32),
                                  _dev(sorted_routes, "sorted_routes", torch.int32),
                                  _dev(route_pos, "route_pos", torch.int32), _stream()), "moe_permute", 2)


LINEAR_PAD_ROWS = 16


# Steps of this many tokens stream the weights with this library's own kernel (0 switches it off).  The
# kernel takes up to four rows, but measured on B200 (3072 x 8192 and 6144 x 3072, inside a decode step) it
# wins against the library's 16-row product only for one: 10.2 / 9.3 against 11.2 / 11.1 microseconds; at
# two rows 12.9 / 14.5, at four 17 / 19.6 (the lanes run out of issue slots, not of bandwidth).
SMALL_LINEAR_MAX_TOKENS = 1


def small_linear_fits(n_tokens: int, n_out: int, k: int) -> bool:
    return bool(_lib().ftk_small_linear_fits(n_tokens, n_out, k))


def small_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ w^T`` in bfloat16 for one to four rows of ``x``: every SM streams its share of the
    weight rows once, 32-bit sums (``csrc/gemv.cu``)."""
    T, K = x.shape
    N = w.shape[0]
    if w.shape != (N, K) or out.shape != (T, N) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 \
            or out.dtype != torch.bfloat16:
        raise KernelError("small_linear: bfloat16 x [T, K], w [N, K], out [T, N] expected")
    _check(_lib().ftk_small_linear(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), T, N, K, _stream()), "small_linear")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ w^T`` (``x [T, K]``, ``w [N, K]``, ``out [T, N]``): by the library, as in the reference
    (python/freetoken/layers/linear.py:66-70), except for bfloat16 steps of up to four tokens, whose
    product is a stream over the weights that :func:`small_linear` does faster than the library's choice
    of tile (measured on B200, 3072 x 8192 for one token: see the design notes).

    For fewer than 16 rows of bfloat16 and a weight that is at least as long as it is tall, the
    product is taken over 16 rows of the same buffers (the rows past ``T`` hold whatever the
    buffers hold and their results are never read): measured on B200, the library's choice for 16
    rows runs 3072 x 6144 in 10.9 microseconds, its choice for 8 rows in 16.6."""
    T, K = x.shape
    N = w.shape[0]
    if w.shape != (N, K) or out.shape != (T, N):
        raise KernelError("linear: shapes do not agree")
    if (T <= SMALL_LINEAR_MAX_TOKENS and x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous()
            and w.is_contiguous() and out.is_contiguous() and small_linear_fits(T, N, K)):
        small_linear(x, w, out)
        return
    P = LINEAR_PAD_ROWS
    if (T < P and K >= N and x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous() and out.is_contiguous()
            and _room(x) >= P * K and _room(out) >= P * N):
        torch.matmul(x.as_strided((P, K), (K, 1)), w.t(), out=out.as_strided((P, N), (N, 1)))
    else:
        torch.matmul(x, w.t(), out=out)


def _room(t: torch.Tensor) -> int:
    """Elements from the tensor's first one to the end of its storage."""
    return t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()


def moe_route_fits(n_tokens: int, hidden: int, n_experts: int, top_k: int) -> bool:
    """Whether :func:`moe_route` takes these sizes (small steps only)."""
    return bool(_lib().ftk_moe_route_fits(n_tokens, hidden, n_experts, top_k))


def moe_route(x: torch.Tensor, gate_w: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, scoring: str,
              scale: float, logits: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
              expert_counts: Optional[torch.Tensor] = None, expert_offsets: Optional[torch.Tensor] = None,
              sorted_routes: Optional[torch.Tensor] = None, route_pos: Optional[torch.Tensor] = None) -> None:
    """``logits = x @ gate_w^T`` in float32, then :func:`router_topk` and :func:`moe_permute`, in one launch.
    Without the four outputs of the sort only ids and weights are made (the few-token expert kernels take
    the routes in token order)."""
    T, H = x.shape
    E = gate_w.shape[0]
    if gate_w.shape != (E, H) or logits.shape != (T, E) or ids.shape != (T, top_k) or weights.shape != (T, top_k):
        raise KernelError("moe_route: shapes do not agree")
    sort = expert_counts is not None
    if sort and (expert_offsets is None or sorted_routes is None or route_pos is None):
        raise KernelError("moe_route: give all four outputs of the sort, or none")
    if sort and (expert_offsets.shape != (E + 1,) or expert_counts.shape != (E,) or sorted_routes.numel() != T * top_k
                 or route_pos.numel() != T * top_k):
        raise KernelError("moe_route: output shapes are wrong")
    if bias is not None and bias.shape != (E,):
        raise KernelError("moe_route: bias must be [E]")
    _check(_lib().ftk_moe_route(_dev(x, "x", torch.float32), _dev(gate_w, "gate_w", torch.float32),
                                _dev(bias, "bias", torch.float32), T, H, E, top_k, SCORE_CODES[scoring], float(scale),
                                _dev(logits, "logits", torch.float32), _dev(ids, "ids", torch.int32),
                                _dev(weights, "weights", torch.float32),
                                _dev(expert_counts, "expert_counts", torch.int32),
                                _dev(expert_offsets, "expert_offsets", torch.int32),
                                _dev(sorted_routes, "sorted_routes", torch.int32),
                                _dev(route_pos, "route_pos", torch.int32), 1 if sort else 0, _stream()), "moe_route")


def moe_small_fits(n_tokens: int, hidden: int, inter: int, top_k: int) -> bool:
    """Whether the few-token expert kernels (:func:`moe_small_gate_up`, :func:`moe_small_down`) take a step."""
    return bool(_lib().ftk_moe_small_fits(n_tokens, hidden, inter, top_k))


def moe_small_gate_up(h: torch.Tensor, ids: torch.Tensor, w1: torch.Tensor, act: str, alpha: float, limit: float,
                      out: torch.Tensor) -> None:
    """``out[t*k + j] = act(h[t] W1[ids[t, j]]^T)`` for a step of up to four tokens: routes in token order,
    no sort, no gathered copy; ``w1 [E, 2I, H]`` rows gate then up, bfloat16."""
    T, H = h.shape
    k = ids.shape[1]
    E, two_i, H2 = w1.shape
    if H2 != H or ids.shape != (T, k) or out.shape != (T * k, two_i // 2) or h.dtype != torch.bfloat16 \
            or w1.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("moe_small_gate_up: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_small_gate_up(_dev(h, "h"), _dev(ids, "ids", torch.int32), _dev(w1, "w1"), _dev(out, "out"),
                                        T, k, E, H, two_i // 2, ACT_CODES[act], float(alpha), float(limit), _stream()),
           "moe_small_gate_up")


def moe_small_down(a: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w2: torch.Tensor,
                   out: torch.Tensor) -> None:
    """``out[r] = (a[r] W2[ids.flat[r]]^T) * weights.flat[r]`` for the routes of up to four tokens.
    ``ids`` are read while the launch before this one may still run (they are the routing kernel's, which
    ended before :func:`moe_small_gate_up` began): a caller that writes them just before must do so with an
    ordinary launch."""
    R, I = a.shape
    E, H, I2 = w2.shape
    T, k = ids.shape
    if I2 != I or R != T * k or weights.numel() != R or out.shape != (R, H) or a.dtype != torch.bfloat16 \
            or w2.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("moe_small_down: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_small_down(_dev(a, "a"), _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32),
                                     _dev(w2, "w2"), _dev(out, "out"), T, k, E, H, I, _stream()), "moe_small_down")


def moe_gather(h: torch.Tensor, sorted_routes: torch.Tensor, top_k: int, out: torch.Tensor) -> None:
    """``out[r, :] = h[sorted_routes[r] // top_k, :]``."""
    T, H = h.shape
    R = sorted_routes.numel()
    if out.shape != (R, H) or out.dtype != h.dtype:
        raise KernelError("moe_gather: out must be [routes, hidden] of h's dtype")
    _check(_lib().ftk_moe_gather(_dev(h, "h"), _code(h, "h"), _dev(sorted_routes, "sorted_routes", torch.int32),
                                 R, top_k, H, _dev(out, "out"), _stream()), "moe_gather")


def moe_gemm1_act(x_sorted: torch.Tensor, w1: torch.Tensor, expert_offsets: torch.Tensor,
                  act: str, alpha: float, limit: float, out: torch.Tensor) -> None:
    """``out[r] = act(x[r] W1[e]^T)`` for the rows of each expert; ``w1 [E, 2I, H]`` rows gate then up."""
    R, H = x_sorted.shape
    E, two_i, H2 = w1.shape
    if H2 != H or two_i % 2 or out.shape != (R, two_i // 2) or w1.dtype != x_sorted.dtype \
            or out.dtype != x_sorted.dtype:
        raise KernelError("moe_gemm1_act: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_gemm1_act(_dev(x_sorted, "x_sorted"), _dev(w1, "w1"), _code(w1, "w1"),
                                    _dev(expert_offsets, "expert_offsets", torch.int32), E, R, H,
                                    two_i // 2, ACT_CODES[act], float(alpha), float(limit),
                                    _dev(out, "out"), _stream()), "moe_gemm1_act")


def moe_gemm1_gather_fits(dtype: torch.dtype, hidden: int, inter: int, n_experts: int, n_routes: int) -> bool:
    """Whether :func:`moe_gemm1_act_gather` takes these sizes (bfloat16 on the tensor cores, few enough routes
    per expert for token tiles of at most 32 rows)."""
    return dtype == torch.bfloat16 and bool(_lib().ftk_moe_gemm1_gather_fits(hidden, inter, n_experts, n_routes))


def moe_gemm1_act_gather(h: torch.Tensor, sorted_routes: torch.Tensor, top_k: int, w1: torch.Tensor,
                         expert_offsets: torch.Tensor, act: str, alpha: float, limit: float, out: torch.Tensor) -> None:
    """:func:`moe_gather` and :func:`moe_gemm1_act` in one kernel: ``out[r] = act(h[sorted_routes[r] // top_k]
    W1[e]^T)`` for the rows ``r`` of each expert; ``h [T, H]`` holds the tokens in their own order."""
    T, H = h.shape
    E, two_i, H2 = w1.shape
    R = sorted_routes.numel()
    if H2 != H or two_i % 2 or out.shape != (R, two_i // 2) or w1.dtype != h.dtype or out.dtype != h.dtype \
            or h.dtype != torch.bfloat16 or R != T * top_k or not h.is_contiguous():
        raise KernelError("moe_gemm1_act_gather: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_gemm1_act_gather(_dev(h, "h"), _dev(w1, "w1"),
                                           _dev(expert_offsets, "expert_offsets", torch.int32),
                                           _dev(sorted_routes, "sorted_routes", torch.int32), int(top_k), T, E, R, H,
                                           two_i // 2, ACT_CODES[act], float(alpha), float(limit),
                                           _dev(out, "out"), _stream()), "moe_gemm1_act_gather")


def moe_gemm2(a: torch.Tensor, w2: torch.Tensor, expert_offsets: torch.Tensor,
              sorted_routes: torch.Tensor, topk_weights: torch.Tensor, out: torch.Tensor) -> None:
    """``out[r] = (a[r] W2[e]^T) * topk_weights[sorted_routes[r]]``; ``w2 [E, H, I]``."""
    R, I = a.shape
    E, H, I2 = w2.shape
    if I2 != I or out.shape != (R, H) or w2.dtype != a.dtype or out.dtype != a.dtype:
        raise KernelError("moe_gemm2: shapes or dtypes do not agree")
    if topk_weights.numel() != R or sorted_routes.numel() != R:
        raise KernelError("moe_gemm2: one weight and one route per row expected")
    _check(_lib().ftk_moe_gemm2(_dev(a, "a"), _dev(w2, "w2"), _code(w2, "w2"),
                                _dev(expert_offsets, "expert_offsets", torch.int32),
                                _dev(sorted_routes, "sorted_routes", torch.int32),
                                _dev(topk_weights, "topk_weights", torch.float32), E, R, H, I,
                                _dev(out, "out"), _stream()), "moe_gemm2")


def moe_combine(y: torch.Tensor, route_pos: torch.Tensor, n_tokens: int, top_k: int,
                shared: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out[t] = sum_j y[route_pos[t*k + j]]`` in route order, 32-bit sum, ``+ shared[t]``."""
    R, H = y.shape
    if R != n_tokens * top_k or out.shape != (n_tokens, H) or out.dtype != y.dtype:
        raise KernelError("moe_combine: shapes or dtypes do not agree")
    if shared is not None and (shared.shape != out.shape or shared.dtype != y.dtype):
        raise KernelError("moe_combine: shared must match out")
    _check(_lib().ftk_moe_combine(_dev(y, "y"), _code(y, "y"), _dev(route_pos, "route_pos", torch.int32),
                                  n_tokens, top_k, H, _dev(shared, "shared"), _dev(out, "out"),
                                  _stream()), "moe_combine")


# --------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           u: torch.Tensor, out: torch.Tensor) -> None:
    """One token per row of float32 ``logits [R, V]``.

    ``temperature[r] <= 0``: argmax, lowest index on a tie.  Else ``p = softmax(logits / T)``;
    top-k keeps ``p >=`` the k-th largest value (``top_k <= 0`` keeps all); top-p then keeps
    ``p >= th`` for the largest ``th`` whose kept mass reaches ``top_p`` of the remaining mass;
    the token is the first index whose running kept mass exceeds ``u[r]`` times the kept mass.
    """
    R, V = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("u", u, torch.float32),
                        ("out", out, torch.int32)):
        if t.numel() < R:
            raise KernelError(f"sample: {name} has fewer than {R} entries")
    _check(_lib().ftk_sample(_dev(logits, "logits", torch.float32), R, V,
                             _dev(temperature, "temperature", torch.float32),
                             _dev(top_k, "top_k", torch.int32), _dev(top_p, "top_p", torch.float32),
                             _dev(u, "u", torch.float32), _dev(out, "out", torch.int32), _stream()),
           "sample")
