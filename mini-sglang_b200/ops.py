"""Python face of the engine's CUDA kernels.

Every function here launches hand-written sm_100a kernels from `csrc/` on the current CUDA
stream of torch and returns torch tensors.  There is no other implementation behind them: a
tensor that is not on a CUDA device, a missing compiler or an unsupported size raises.
Matrix products with more than a few rows are the one exception to "hand-written": `linear` then calls
the library GEMM that torch binds (cuBLAS), in bfloat16 with float32 accumulation or in true float32
(TF32 off), as the reference does for every projection (F.linear in mini_sglang/layers/linear.py).  Up to
SMALL_M_MAX rows go to this engine's weight-streaming kernel.  The reference's own kernels for the
other operations come from sgl_kernel / flash-attn (mini_sglang/layers/layernorm.py:39-50,
mini_sglang/layers/rotary_embedding.py, mini_sglang/layers/attn/fa3_attn_backend.py).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence, Tuple

import torch

from .csrc import build as _build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_ERR = {1: "element type not handled", 2: "size not supported by the kernel", 3: "kernel launch failed",
        4: "pointer not aligned"}

c_void_p, c_int, c_float, c_ll, c_ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong


class KernelError(RuntimeError):
    pass


LAUNCHES = 0      # kernels of this engine launched (or recorded into a graph) so far


def _check(code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        detail = ""
        if code == 3:
            detail = f" ({torch.cuda.get_device_name()}: the kernels are built for sm_100a only)"
        raise KernelError(f"{what}: {_ERR.get(code, f'error {code}')}{detail}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr()


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's kernels run on a CUDA device only; got a tensor on " + str(t.device))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not handled; the engine computes in bfloat16 or float32") from None


_common = None
_attn = {}


def _lib():
    global _common
    if _common is None:
        lib = _build.common_library()
        lib.msgl_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_resolve_ids.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.msgl_table_delta.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p]
        lib.msgl_decode_meta.argtypes = [c_void_p] * 4 + [c_int, c_int, c_void_p, c_int, c_int, c_int, c_int] + [c_void_p] * 9 + [c_int, c_void_p, c_void_p, c_void_p, c_int,
                                         c_void_p]
        lib.msgl_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p,
                                     c_int, c_int, c_int, c_void_p]
        lib.msgl_qknorm_rope_kvwrite.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_float, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_swiglu.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.msgl_cast_from_f32.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_void_p]
        lib.msgl_gemm_small_m.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_int,
                                          c_int, c_void_p]
        lib.msgl_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_int, c_void_p,
                                     c_void_p]
        lib.msgl_gemm_tc2.argtypes = lib.msgl_gemm_tc.argtypes
        lib.msgl_gemm_tc2_splitk.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int,
                                             c_void_p, c_void_p, c_void_p]
        lib.msgl_gemm_tc2_splits.argtypes = [c_int, c_int, c_int, c_int]
        lib.msgl_gemm_tc2_splits.restype = c_int
        lib.msgl_sample.argtypes = [c_void_p, c_int, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_ull, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        _common = lib
    return _common


def _attn_lib(head_dim: int):
    hd = head_dim if head_dim in _build.MMA_HEAD_DIMS else 128
    lib = _attn.get(hd)
    if lib is None:
        lib = _build.attention_library(hd)
        lib.msgl_attention.argtypes = [c_void_p] * 10 + [c_int] * 9 + [c_float] + [c_int] * 6 + [c_void_p, c_void_p, c_int, c_void_p]
        lib.msgl_attention_window.argtypes = [c_void_p] * 10 + [c_int] * 9 + [c_float] + [c_int] * 6 + [c_void_p, c_int, c_void_p, c_int, c_void_p]
        lib.msgl_attention_combine.argtypes = [c_void_p] * 5 + [c_int] * 5 + [c_void_p]
        lib.msgl_attention_tc.argtypes = [c_void_p] * 7 + [c_int] * 8 + [c_float] + [c_int] * 5 + [c_void_p, c_int, c_void_p, c_int, c_void_p]
        lib.msgl_attention_head_dim.restype = c_int
        _attn[hd] = lib
    return lib


def warm_up(head_dims=()) -> None:
    """Build and load the libraries a model needs (compiles at the first call)."""
    _lib()
    for hd in head_dims:
        _attn_lib(hd)


# ---------------------------------------------------------------------------------------

def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ids int32 [T], table [V, H] -> float32 [T, H] (the residual stream starts in float32)."""
    _need_cuda(ids, table)
    T, (V, H) = ids.numel(), table.shape
    assert ids.dtype == torch.int32 and table.is_contiguous()
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(_lib().msgl_embedding(_ptr(ids), _ptr(table), _ptr(out), T, H, V, _dt(table), _stream()), "embedding")
    return out


def resolve_ids(ids: torch.Tensor, prev: torch.Tensor) -> None:
    """In place: ids[t] = prev[-1 - ids[t]] where ids[t] < 0 (int32, on the device)."""
    _need_cuda(ids, prev)
    assert ids.dtype == torch.int32 and prev.dtype == torch.int32 and ids.is_contiguous() and prev.is_contiguous()
    _check(_lib().msgl_resolve_ids(_ptr(ids), _ptr(prev), ids.numel(), prev.numel(), _stream()), "resolve_ids")


def table_delta(deltas: torch.Tensor, n_records: int, table: torch.Tensor) -> None:
    """Rows of the device copy of a cache group's block tables, brought up to date: deltas = [n, (slot, count, offset) x n,
    page ids ...] int32 on the device; table int32 [slots, pages per request]."""
    _need_cuda(deltas, table)
    assert deltas.dtype == torch.int32 and table.dtype == torch.int32 and table.is_contiguous()
    _check(_lib().msgl_table_delta(_ptr(deltas), n_records, _ptr(table), table.shape[1], _stream()), "table_delta")


def decode_meta(ids: torch.Tensor, slots_in: torch.Tensor, pos: torch.Tensor, nsplit_in: torch.Tensor, B: int, b: int,
                table: torch.Tensor, page_size: int, mp: int, common: bool, *, input_ids, positions, token_req, q_start, kv_len,
                slots, out_loc, nsplit, block_table, order, window: int = 0, even_in: Optional[torch.Tensor] = None,
                even_out: Optional[torch.Tensor] = None) -> None:
    """The step fields of a decode batch of B requests (captured size b) written on the device from (token id, slot,
    position) per request and the device copy of the block tables; see csrc/elementwise.cu.  `order` receives the rows
    by falling number of keys per kv split (what the attention launch walks first); `even_in` (the even cut of the step's
    keys, made by the host) is copied to `even_out` as it is."""
    _need_cuda(ids, slots_in, pos, nsplit_in, table, input_ids, block_table)
    code = _lib().msgl_decode_meta(_ptr(ids), _ptr(slots_in), _ptr(pos), _ptr(nsplit_in), B, b, _ptr(table), table.shape[1], page_size,
                                   mp, int(common), _ptr(input_ids), _ptr(positions), _ptr(token_req), _ptr(q_start), _ptr(kv_len),
                                   _ptr(slots), _ptr(out_loc), _ptr(nsplit), _ptr(block_table), int(window), _ptr(order),
                                   _ptr(even_in), _ptr(even_out), even_in.numel() if even_in is not None else 0, _stream())
    _check(code, "decode_meta")


def rmsnorm(weight: torch.Tensor, eps: float, *, x: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(residual + x) * weight, the sum and the norm in float32.

    x: activation dtype [N, H] or None; residual: float32 [N, H] or None; residual_out: float32
    buffer that receives the sum (may be `residual` itself when `rows` is None);
    rows: int32 [R] picks input rows (outputs are then [R, H]).  Returns y in `out_dtype`
    (default: x's dtype)."""
    _need_cuda(weight, x, residual, residual_out, rows)
    src = x if x is not None else residual
    assert src is not None and src.dim() == 2 and src.is_contiguous()
    H = src.shape[1]
    n_out = rows.numel() if rows is not None else src.shape[0]
    if out_dtype is None:
        out_dtype = x.dtype if x is not None else torch.float32
    if x is not None:
        assert x.dtype == out_dtype
    if residual is not None:
        assert residual.dtype == torch.float32 and residual.shape[1] == H
    assert weight.numel() == H and weight.dtype in (torch.float32, torch.bfloat16)
    if out is None:
        out = torch.empty((n_out, H), dtype=out_dtype, device=src.device)
    code = _lib().msgl_rmsnorm(_ptr(x), _ptr(residual), _ptr(residual_out), _ptr(rows), _ptr(weight),
                               int(weight.dtype == torch.float32), float(eps), _ptr(out), n_out, H, _DT[out_dtype],
                               _stream())
    _check(code, "rmsnorm")
    return out


def qknorm_rope_kvwrite(qkv: torch.Tensor, positions: torch.Tensor, n_q: int, n_kv: int, d: int, *,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        rope_table: Optional[torch.Tensor], out_loc: Optional[torch.Tensor],
                        k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], page_size: int,
                        q_out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """Per-head RMSNorm of q and k (if weights are given), rotary encoding from `rope_table`
    [max_pos, rot] float32 = cos | sin (if given; the first `rot` elements of a head are rotated in halves, element i
    against i + rot/2, or with `interleaved` in neighbouring pairs 2p, 2p+1), k and v written to the paged cache at token
    slots `out_loc` (if a cache is given), q returned as [T, n_q, d]."""
    _need_cuda(qkv, positions, q_weight, k_weight, rope_table, out_loc, k_cache, v_cache)
    T = qkv.shape[0]
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (n_q + 2 * n_kv) * d
    assert positions.numel() == T and positions.dtype == torch.int32
    if out_loc is not None:
        assert out_loc.numel() == T and out_loc.dtype == torch.int32, "one cache slot per token"
    if q_out is None:
        q_out = torch.empty((T, n_q, d), dtype=qkv.dtype, device=qkv.device)
    w_f32 = 0
    if q_weight is not None:
        assert k_weight is not None and q_weight.dtype == k_weight.dtype
        w_f32 = int(q_weight.dtype == torch.float32)
    rot, max_pos = (rope_table.shape[1], rope_table.shape[0]) if rope_table is not None else (0, 0)
    if rope_table is not None:
        assert rope_table.dtype == torch.float32 and rope_table.is_contiguous()
    if k_cache is not None:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    code = _lib().msgl_qknorm_rope_kvwrite(_ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(out_loc), _ptr(q_weight),
                                           _ptr(k_weight), w_f32, float(eps), _ptr(rope_table), rot, max_pos,
                                           _ptr(q_out), _ptr(k_cache), _ptr(v_cache), page_size, n_q, n_kv, d, T,
                                           _dt(qkv), int(bool(interleaved)), _stream())
    _check(code, f"qknorm_rope_kvwrite (head size {d})")
    return q_out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[T, 2I] (gate first) -> [T, I] = silu(gate) * up."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    T, I = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    _check(_lib().msgl_swiglu(_ptr(gate_up), _ptr(out), T, I, _dt(gate_up), _stream()), "swiglu")
    return out


def cast_from_f32(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(_lib().msgl_cast_from_f32(_ptr(x), _ptr(out), x.numel(), _DT[dtype], _stream()), "cast")
    return out


_sample_scratch = {}          # per device: (part, row_max, tickets)
_sm_counts = {}


def sm_count(device) -> int:
    """Number of SMs of a CUDA device (asked once)."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _sm_counts:
        _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_counts[idx]



def _sample_buffers(device, rows: int, slices: int):
    """Scratch of the sampling kernels, kept per device and grown on demand.  The tickets are zero between calls:
    the block that takes a row's last ticket puts it back to zero."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    part, row_max, tickets = _sample_scratch.get(key, (None, None, None))
    if part is None or part.numel() < rows * slices * 2 or tickets.numel() < rows:
        n_rows = max(rows, 256, tickets.numel() if tickets is not None else 0)
        part = torch.empty(max(rows * slices * 2, 256 * 64 * 2), dtype=torch.float32, device=device)
        row_max = torch.empty(n_rows, dtype=torch.float32, device=device)
        tickets = torch.zeros(n_rows, dtype=torch.int32, device=device)
        _sample_scratch[key] = (part, row_max, tickets)
    return part, row_max, tickets


def sample(logits: torch.Tensor, temperatures: Optional[torch.Tensor], row_keys: Optional[torch.Tensor],
           steps: Optional[torch.Tensor], seed: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 logits [N, V] -> int32 token ids [N]; greedy where temperature is 0."""
    _need_cuda(logits, temperatures, row_keys, steps)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    N, V = logits.shape
    if out is None:
        out = torch.empty((N,), dtype=torch.int32, device=logits.device)
    if N == 0:
        return out
    if temperatures is not None:
        assert temperatures.dtype == torch.float32 and row_keys.dtype == torch.int32 and steps.dtype == torch.int32
    # blocks per row: about four blocks an SM over all rows, but no slice below 2,048 entries
    sms = sm_count(logits.device)
    slices = max(1, min(-(-4 * sms // N), V // 2048, 64))
    part, row_max, tickets = _sample_buffers(logits.device, N, slices)
    code = _lib().msgl_sample(_ptr(logits), N, V, logits.stride(0), _ptr(temperatures), _ptr(row_keys), _ptr(steps),
                              seed & 0xFFFFFFFFFFFFFFFF, _ptr(out), _ptr(part), _ptr(row_max), _ptr(tickets), slices, _stream())
    _check(code, "sample")
    if temperatures is not None:
        global LAUNCHES
        LAUNCHES += 1            # the race is a kernel of its own
    return out


# ---------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------
VARIANT_SIMT, VARIANT_MMA_ROWS, VARIANT_MMA_DECODE, VARIANT_TC = 0, 1, 2, 3
TC_ROWS = 128                     # query rows per block of the tcgen05 prefill kernel
USE_TC_ATTENTION = os.environ.get("MSGL_NO_TC_ATTENTION", "") == ""
_status = None                    # device int32[64]: word 0 tcgen05 attention, word 2 tcgen05 GEMM, word 3 decode-step kernel; words 4..: debug counters
_status_host = None               # its pinned mirror, refreshed by poll_status()
_status_event = None


def _status_tensor(device) -> torch.Tensor:
    global _status, _status_host
    if _status is None:
        _status = torch.zeros(64, dtype=torch.int32, device=device)
        _status_host = torch.zeros(64, dtype=torch.int32).pin_memory()
    return _status


def poll_status() -> None:
    """Queue a copy of the kernels' status words to the host (no synchronisation).  Not inside a stream capture."""
    global _status_event
    if _status is None:
        return
    _status_host.copy_(_status, non_blocking=True)
    _status_event = torch.cuda.Event()
    _status_event.record()


def raise_if_failed(wait: bool = False) -> None:
    """Raise if a kernel with bounded waits gave up in a launch that the last finished poll_status() saw."""
    if _status_event is None:
        return
    if wait:
        _status_event.synchronize()
    elif not _status_event.query():
        return
    if int(_status_host[0]) != 0:
        raise KernelError("tcgen05 attention: a block timed out waiting for the tensor core; results are invalid")
    if int(_status_host[2]) != 0:
        raise KernelError("tcgen05 GEMM: a block timed out waiting for its pipeline; results are invalid")
    if int(_status_host[3]) != 0:
        raise KernelError("decode step: a block timed out at a grid barrier; results are invalid")


def tc_supported(head_dim: int, dtype: torch.dtype, group: int) -> bool:
    """The tcgen05 prefill attention kernels take bfloat16, head size 128, up to 128 query heads per kv head."""
    return USE_TC_ATTENTION and dtype == torch.bfloat16 and head_dim == 128 and 1 <= group <= TC_ROWS


def check_kernel_status() -> None:
    """Raise if a block of a kernel with bounded waits ever gave up waiting (synchronises)."""
    poll_status()
    raise_if_failed(wait=True)


TC_VERSION = int(os.environ.get("MSGL_TC_VERSION", "2"))      # 2: two query tiles per block in ping-pong (needs TMA page sizes); 1: one tile
_tc2_usable = True


def attention_tc(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                 q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, n_kv: int, page_size: int,
                 window: int, scale: float, qlen_min: int, qlen_max: int, q_lens: Sequence[int], keep_first: int = 0,
                 bias_log2: Optional[torch.Tensor] = None) -> bool:
    """Prefill attention on tcgen05 tensor cores for the requests with q_len in [qlen_min, qlen_max];
    q_lens: the host's copy of every request's number of query tokens (to size the grid).  keep_first, bias_log2: as in
    `attention`; they are taken by the kernel on pairs of query tiles only (TMA page sizes), and the call returns False,
    having launched nothing, where that kernel cannot run."""
    global _tc2_usable
    _need_cuda(q, out, k_cache, v_cache, q_start, kv_len, block_table)
    T, n_q, d = q.shape
    B = kv_len.numel()
    assert q.is_contiguous() and out.is_contiguous() and block_table.stride(1) == 1 and q.dtype == torch.bfloat16
    status = _status_tensor(q.device)
    group = n_q // n_kv
    whole = k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    pages = k_cache.shape[0] if whole else 0
    tma_pages = whole and page_size >= 8 and (page_size & (page_size - 1)) == 0
    versions = [2, 1] if (TC_VERSION == 2 and _tc2_usable and tma_pages) else [1]
    ext = bool(keep_first) or bias_log2 is not None
    if ext:
        _need_cuda(bias_log2)
        if versions[0] != 2:
            return False
        versions = [2]
        if bias_log2 is not None:
            assert bias_log2.dtype == torch.float32 and bias_log2.dim() == 2 and bias_log2.shape[0] == n_q and bias_log2.is_contiguous()
    for version in versions:
        rows = TC_ROWS * version
        qt = rows // group if group <= TC_ROWS else version
        grid_x = sum(-(-n // qt) for n in q_lens if qlen_min <= n <= qlen_max)
        code = _attn_lib(d).msgl_attention_tc(
            _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table), B, T, n_q,
            n_kv, d, page_size, block_table.stride(0), window, float(scale), qlen_min, qlen_max, grid_x, pages, version,
            _ptr(status), int(keep_first), _ptr(bias_log2), bias_log2.shape[1] if bias_log2 is not None else 0, _stream())
        if code == 2 and version == 2:        # no tensor maps here (driver without the encoder, unaligned cache): one-tile kernel
            _tc2_usable = False
            if ext:
                return False
            continue
        _check(code, "attention_tc")
        return True
    return False


def attention_tile_tokens(variant: int, group: int, head_dim: int = 128) -> int:
    """Tokens per query tile of a kernel variant for a given group size (q heads per kv head)."""
    if variant == VARIANT_MMA_DECODE:
        lib = _attn_lib(head_dim)
        lib.msgl_attention_decode_tile_tokens.restype = c_int
        return int(lib.msgl_attention_decode_tile_tokens(int(group)))
    rows = {VARIANT_MMA_ROWS: 64, VARIANT_TC: TC_ROWS}.get(variant, 16)
    return rows // group if group <= rows else 1


def decode_blocks_per_sm(head_dim: int, dtype: torch.dtype, group: int = 1) -> int:
    """Blocks of the decode attention kernel that fit one SM (used to choose the kv splits)."""
    if not mma_supported(head_dim, dtype):
        return 4
    lib = _attn_lib(head_dim)
    lib.msgl_attention_decode_blocks_per_sm.restype = c_int
    return int(lib.msgl_attention_decode_blocks_per_sm(int(group)))


def even_cut_size(B: int, n_blocks: int) -> int:
    """int32 words of the even cut of a decode step of B requests over n_blocks blocks per kv head: blocks in use, start
    unit of every block [n_blocks + 1], first request of every block [n_blocks], first unit of every request [B + 1], first
    block of every request [B]."""
    return 1 + (n_blocks + 1) + n_blocks + (B + 1) + B


def decode_even_ok(head_dim: int, dtype: torch.dtype, group: int = 1) -> bool:
    """Whether the decode attention launch for this head size takes an even cut of the keys (`attention(even=...)`)."""
    if not mma_supported(head_dim, dtype):
        return False
    lib = _attn_lib(head_dim)
    lib.msgl_attention_decode_even_ok.restype = c_int
    return bool(lib.msgl_attention_decode_even_ok(int(group)))


def window_bias_supported(head_dim: int, dtype: torch.dtype, group: int) -> bool:
    """Whether `attention(keep_first=..., bias_log2=...)` takes this geometry: bfloat16, head sizes in steps of 32 (the mma
    prefill kernel and the transposed decode kernel), up to 16 query heads a kv head."""
    return mma_supported(head_dim, dtype) and head_dim % 32 == 0 and group <= 16


def mma_supported(head_dim: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and head_dim in _build.MMA_HEAD_DIMS


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
              q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor,
              nsplit: Optional[torch.Tensor], part_o: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
              n_kv: int, page_size: int, window: int, max_split: int, scale: float, qlen_min: int, qlen_max: int,
              uniform_decode: bool, variant: int, grid_x: int, order: Optional[torch.Tensor] = None,
              even: Optional[torch.Tensor] = None, even_nb: int = 0, keep_first: int = 0,
              bias_log2: Optional[torch.Tensor] = None) -> None:
    """One launch of the paged attention kernel over the requests whose q_len lies in
    [qlen_min, qlen_max]; see csrc/attention.cu for the meaning of every argument.  keep_first: with a window, the first
    keys of a request that stay visible whatever the window; bias_log2: float32 [heads, L], added to the scaled score in
    log2 units by distance min(i - j, L - 1) (both: the bfloat16 mma kernels only, see `window_bias_supported`).  `order` (uniform decode only):
    int32 [B], a permutation of the requests; the launch's i-th block along x takes request order[i].  `even`: the even cut
    of a decode step's keys over `even_nb` blocks per kv head (engine/step.py: plan_even_cut) in place of `grid_x` blocks."""
    _need_cuda(q, out, k_cache, v_cache, q_start, kv_len, block_table, nsplit, part_o, part_ml, order, even)
    T, n_q, d = q.shape
    B = kv_len.numel()
    assert q.is_contiguous() and out.is_contiguous() and block_table.dim() == 2 and block_table.stride(1) == 1
    assert q_start.numel() == B + 1 and block_table.shape[0] == B and out.shape == q.shape
    assert nsplit is None or nsplit.numel() == B
    assert order is None or (uniform_decode and order.numel() == B and order.dtype == torch.int32)
    assert even is None or (uniform_decode and variant == VARIANT_MMA_DECODE and even.dtype == torch.int32 and
                            even.numel() >= even_cut_size(B, even_nb) and even_nb >= 1)
    if max_split > 1:
        assert part_o.numel() >= max_split * T * n_q * d and part_ml.numel() >= max_split * T * n_q * 2
    if keep_first or bias_log2 is not None:
        _need_cuda(bias_log2)
        assert even is None, "the even cut of a decode step knows no kept tokens and no bias"
        if bias_log2 is not None:
            assert bias_log2.dtype == torch.float32 and bias_log2.dim() == 2 and bias_log2.shape[0] == n_q and bias_log2.is_contiguous()
        code = _attn_lib(d).msgl_attention_window(
            _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table),
            _ptr(nsplit), _ptr(part_o), _ptr(part_ml), B, T, n_q, n_kv, d, page_size, block_table.stride(0), window,
            max_split, float(scale), qlen_min, qlen_max, int(uniform_decode), variant, grid_x, _dt(q), _ptr(order),
            int(keep_first), _ptr(bias_log2), bias_log2.shape[1] if bias_log2 is not None else 0, _stream())
        _check(code, f"attention with kept tokens / bias (head size {d}, variant {variant})")
        return
    code = _attn_lib(d).msgl_attention(
        _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table),
        _ptr(nsplit), _ptr(part_o), _ptr(part_ml), B, T, n_q, n_kv, d, page_size, block_table.stride(0), window,
        max_split, float(scale), qlen_min, qlen_max, int(uniform_decode), variant, grid_x, _dt(q), _ptr(order), _ptr(even), int(even_nb), _stream())
    _check(code, f"attention (head size {d}, variant {variant})")


def attention_combine(part_o: torch.Tensor, part_ml: torch.Tensor, token_req: Optional[torch.Tensor],
                      nsplit: torch.Tensor, out: torch.Tensor, max_split: int) -> None:
    _need_cuda(part_o, part_ml, token_req, nsplit, out)
    T, n_q, d = out.shape
    code = _attn_lib(d).msgl_attention_combine(_ptr(part_o), _ptr(part_ml), _ptr(token_req), _ptr(nsplit), _ptr(out),
                                               T, n_q, d, max_split, _dt(out), _stream())
    _check(code, "attention_combine")


# ---------------------------------------------------------------------------------------
# matrix products: the library GEMM (cuBLAS through torch)
# ---------------------------------------------------------------------------------------

def set_true_fp32() -> None:
    """float32 products are real float32: no TF32, no reduced-precision reduction."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.set_float32_matmul_precision("highest")


SMALL_M_MAX = int(os.environ.get("MSGL_SMALL_M_MAX", "8"))      # tokens up to which the weight-streaming kernel replaces the library GEMM (measured: faster up to 8)
USE_SMALL_M = os.environ.get("MSGL_NO_SMALL_M", "") == ""


def _small_m(weight, x, bias, out, M, N, K, ldo, mode, out_f32) -> int:
    return _lib().msgl_gemm_small_m(_ptr(weight), _ptr(x), _ptr(bias), _ptr(out), M, N, K, x.stride(0), ldo, mode, out_f32, _stream())


def _small_m_ok(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> bool:
    return (USE_SMALL_M and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= SMALL_M_MAX and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and weight.shape[1] % 32 == 0 and weight.shape[0] % 16 == 0
            and (bias is None or bias.dtype == torch.bfloat16))


# This engine's tcgen05 GEMM (csrc/gemm_tc.cu) against the library's, measured on B200 at Qwen3-8B's sizes.  With SwiGLU in
# its epilogue the kernel on pairs of SMs (cta_group::2) beats library GEMM + activation kernel from about 256 rows on
# (512 rows: 83 against 86 us, 2,048 rows: 285 against 310 us, 4,096 rows: 0.52 against 0.72 ms; 2,048-token prefill step
# 27.4 -> 26.4 ms).  Its plain products reach 92-95 % of the library's speed at 2,048 rows (the one-block kernel: 88 %), so
# those stay with the library unless MSGL_TC_GEMM=all (prefill step + 1.3 ms).  MSGL_TC_GEMM=0 switches the kernel off,
# MSGL_TC_GEMM_CTAS=1 takes the one-block kernel.
TC_GEMM = os.environ.get("MSGL_TC_GEMM", "swiglu")            # "swiglu" | "all" | "0"
TC_GEMM_MIN_M = int(os.environ.get("MSGL_TC_GEMM_MIN_M", "256"))
TC_GEMM_CTAS = int(os.environ.get("MSGL_TC_GEMM_CTAS", "2"))   # 2: the kernel on pairs of SMs (tcgen05 cta_group::2)
_tc_gemm_usable = True


def _tc_gemm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], mode: int) -> Optional[torch.Tensor]:
    """x @ weight^T (mode 0) or SwiGLU of it (mode 1) by the tcgen05 kernel; None where it does not apply."""
    global _tc_gemm_usable
    if not ((TC_GEMM == "all" or (TC_GEMM == "swiglu" and mode == 1)) and _tc_gemm_usable and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and x.shape[0] >= TC_GEMM_MIN_M and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and weight.shape[1] % 8 == 0 and (bias is None or bias.dtype == torch.bfloat16)):
        return None
    M, (N, K) = x.shape[0], weight.shape
    n_out = N // 2 if mode == 1 else N
    if n_out % 8 or (mode == 1 and N % 2):
        return None
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    fn = _lib().msgl_gemm_tc2 if TC_GEMM_CTAS == 2 else _lib().msgl_gemm_tc
    code = fn(_ptr(weight), _ptr(x), _ptr(bias), _ptr(out), M, N, K, x.stride(0), n_out, mode, _ptr(_status_tensor(x.device)), _stream())
    if code == 2:             # no tensor maps on this driver
        _tc_gemm_usable = False
        return None
    _check(code, "gemm_tc")
    return out


# Between the weight-streaming kernel (up to SMALL_M_MAX rows) and the tiled tcgen05 kernel (from TC_GEMM_MIN_M rows) a product has
# too few output tiles to fill the GPU: there the pair kernel cuts K into ranges as well (split-K) and a second kernel adds
# the ranges' float32 partial sums in order.  Off unless MSGL_TC_MID=1: measured on B200 at Qwen3-8B's sizes it is behind the
# library GEMM at 16 to 128 rows (qkv 18-26 against 12.5 us, o 15-21 against 10, gate/up + SwiGLU 44-66 against 42-45, down 26-33
# against 21-22 us), so these sizes stay with the library.
MID_GEMM = os.environ.get("MSGL_TC_MID", "0") == "1"
MID_GEMM_SPLITS = int(os.environ.get("MSGL_TC_MID_SPLITS", "0"))        # 0: chosen per size
_mid_partials = {}
_mid_splits = {}


def _tc_gemm_mid(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], mode: int) -> Optional[torch.Tensor]:
    """x @ weight^T (mode 0) or SwiGLU of it (mode 1) for a middling number of rows by the split-K tcgen05 kernel; None where
    it does not apply."""
    global _tc_gemm_usable
    if not (MID_GEMM and TC_GEMM != "0" and TC_GEMM_CTAS == 2 and _tc_gemm_usable and x.dtype == torch.bfloat16
            and weight.dtype == torch.bfloat16 and x.dim() == 2 and SMALL_M_MAX < x.shape[0] < TC_GEMM_MIN_M and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.is_contiguous() and weight.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0
            and weight.shape[1] >= 512 and (bias is None or bias.dtype == torch.bfloat16)):
        return None
    M, (N, K) = x.shape[0], weight.shape
    n_out = N // 2 if mode == 1 else N
    if n_out % 8 or (mode == 1 and N % 16):
        return None
    key = (M, N, K, mode)
    splits = MID_GEMM_SPLITS or _mid_splits.get(key)
    if not splits:
        splits = _mid_splits[key] = int(_lib().msgl_gemm_tc2_splits(M, N, K, mode))
    splits = max(1, min(splits, K // 64))
    part = None
    if splits > 1:
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        part = _mid_partials.get(dev)
        if part is None or part.numel() < splits * M * N:
            part = _mid_partials[dev] = torch.empty(max(splits * M * N, 1 << 22), dtype=torch.float32, device=x.device)
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    code = _lib().msgl_gemm_tc2_splitk(_ptr(weight), _ptr(x), _ptr(bias), _ptr(out), M, N, K, x.stride(0), n_out, mode, splits,
                                       _ptr(part), _ptr(_status_tensor(x.device)), _stream())
    if code == 2:             # no tensor maps on this driver
        _tc_gemm_usable = False
        return None
    _check(code, "gemm_tc (split-K)")
    if splits > 1:
        global LAUNCHES
        LAUNCHES += 1
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x @ weight^T (+ bias); weight is [out, in] as stored in the checkpoint.

    Up to SMALL_M_MAX bfloat16 rows go through this engine's weight-streaming kernel
    (csrc/gemm_small_m.cu); everything else is the library GEMM."""
    _need_cuda(x, weight, bias)
    if _small_m_ok(x, weight, bias) and out_dtype in (None, torch.bfloat16, torch.float32):
        M, (N, K) = x.shape[0], weight.shape
        od = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=od, device=x.device)
        code = _small_m(weight, x, bias, out, M, N, K, N, 0, int(od == torch.float32))
        _check(code, "gemm_small_m")
        return out
    if out_dtype in (None, torch.bfloat16):
        y = _tc_gemm(x, weight, bias, 0) if x.shape[0] >= TC_GEMM_MIN_M else _tc_gemm_mid(x, weight, bias, 0)
        if y is not None:
            return y
    if out_dtype is not None and out_dtype != x.dtype:
        y = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            y += bias.to(out_dtype)
        return y
    return torch.nn.functional.linear(x, weight, bias)


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x @ gate^T) * (x @ up^T) with gate_up = [gate; up] packed row-wise ([2I, H]).  For a few
    rows the product and the activation are one kernel and the [T, 2I] intermediate never exists."""
    _need_cuda(x, gate_up)
    if _small_m_ok(x, gate_up, None) and (gate_up.shape[0] // 2) % 8 == 0:
        M, (N, K) = x.shape[0], gate_up.shape
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        code = _small_m(gate_up, x, None, out, M, N, K, N // 2, 1, 0)
        _check(code, "gemm_small_m (swiglu)")
        return out
    y = _tc_gemm(x, gate_up, None, 1) if x.shape[0] >= TC_GEMM_MIN_M else _tc_gemm_mid(x, gate_up, None, 1)
    if y is not None:
        return y
    return swiglu(torch.nn.functional.linear(x, gate_up))


# ---------------------------------------------------------------------------------------
# norms, convolutions, windowed and linear attention, gated activations (csrc/mixers.cu)
# ---------------------------------------------------------------------------------------
_mixers = None
ACT_SILU, ACT_GELU_TANH, ACT_SIGMOID = 0, 1, 2
WINDOW_ATTENTION_ROWS = 8         # (token, head) rows of a block of the windowed attention kernel
CONV_MAX_TAPS = 16
WINDOW_ATTENTION_MAX_HEAD_DIM = 512
DECAY_ATTENTION_MAX_KEY_DIM = 512


def _mix_lib():
    global _mixers
    if _mixers is None:
        lib = _build.mixers_library()
        lib.msgl_dyntanh.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int,
                                     c_int, c_void_p]
        lib.msgl_conv_norm_kvwrite.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_int] + [c_void_p] * 4 + \
            [c_float] + [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_window_attention.argtypes = [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_ll, c_int,
                                              c_void_p, c_ll, c_int] + [c_int] * 9 + [c_float, c_float, c_int, c_void_p]
        lib.msgl_decay_attention.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int] + [c_void_p] * 5 + \
            [c_int, c_int, c_void_p]
        lib.msgl_rms_gate.argtypes = [c_void_p, c_int, c_void_p, c_float, c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_float, c_int,
                                      c_int, c_void_p]
        lib.msgl_gated_act.argtypes = [c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_head_gate.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
        lib.msgl_decay_attention_chunked.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int] + [c_void_p] * 6 + \
            [c_int, c_int, c_int, c_void_p]
        lib.msgl_scaled_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]
        lib.msgl_postnorm_residual.argtypes = [c_void_p, c_int, c_void_p, c_float, c_float, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                               c_int, c_int, c_void_p]
        lib.msgl_latent_prep.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                         c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.msgl_rope_heads.argtypes = [c_void_p, c_ll, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float,
                                        c_void_p, c_int, c_int, c_void_p]
        lib.msgl_gate_mul.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_gated_decay_attention.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                                   c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.msgl_gated_decay_attention_chunked.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                           c_float, c_float] + [c_void_p] * 7 + [c_int, c_int, c_int, c_void_p]
        lib.msgl_group_rms_gate.argtypes = [c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_ll, c_void_p, c_ll, c_float, c_int,
                                            c_int, c_int, c_void_p]
        _mixers = lib
    return _mixers


def _rows_view(t: torch.Tensor, width: int, what: str) -> int:
    """A [T, width] view into packed rows: unit stride along the row; -> the row stride in elements."""
    assert t.dim() == 2 and t.shape[1] == width and (t.stride(1) == 1 or width == 1), f"{what}: [T, {width}] with unit stride wanted"
    return t.stride(0)


def dyntanh(weight: torch.Tensor, bias: torch.Tensor, alpha: float, *, x: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """y = tanh(alpha * v) * weight + bias with v = residual + x in float32 (either may be None); v goes to `residual_out`
    when it is given; `rows` (int32) picks the rows.  x: float32 or `out_dtype`; weight, bias: float32 [H]."""
    _need_cuda(weight, bias, x, residual, residual_out, rows)
    src = x if x is not None else residual
    assert src is not None and src.dim() == 2 and src.is_contiguous()
    H = src.shape[1]
    assert weight.dtype == torch.float32 and bias.dtype == torch.float32 and weight.numel() == H and bias.numel() == H
    if x is not None:
        assert x.dtype in (torch.float32, out_dtype) and x.is_contiguous()
    if residual is not None:
        assert residual.dtype == torch.float32 and residual.shape[1] == H and residual.is_contiguous()
    n_out = rows.numel() if rows is not None else src.shape[0]
    out = torch.empty((n_out, H), dtype=out_dtype, device=src.device)
    code = _mix_lib().msgl_dyntanh(_ptr(x), int(x is not None and x.dtype == torch.float32), _ptr(residual), _ptr(residual_out),
                                   _ptr(rows), _ptr(weight), _ptr(bias), float(alpha), _ptr(out), n_out, H, _DT[out_dtype], _stream())
    _check(code, "dyntanh")
    return out


def conv_norm_kvwrite(q_in: torch.Tensor, k_in: torch.Tensor, *, n_kv: int, head_dim: int, q_taps: torch.Tensor, k_taps: torch.Tensor,
                      q_norm: torch.Tensor, k_norm: torch.Tensor, eps: float, state: torch.Tensor, token_req: torch.Tensor,
                      q_start: torch.Tensor, slots: torch.Tensor, out_loc: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                      v_cache: Optional[torch.Tensor], page_size: int, one_token: bool = False) -> torch.Tensor:
    """Short causal convolution over time on every channel of q_in [T, Cq] and k_in [T, Ck] (views into one packed
    projection) with taps q_taps [taps, Cq] and k_taps [taps, Ck] (float32, the oldest input's tap first), continued from `state` [slots, taps - 1, Cq + Ck] (the request's last inputs, which the call brings up to
    date), then an RMS norm over the whole of q and of k.  The normed k goes to `k_cache`, the un-normed k to `v_cache`
    (layout [page][kv head][slot][head_dim]) at token slots `out_loc`; the normed q comes back as [T, Cq].  one_token: every
    request brings exactly one token (the state is then brought up to date by the same launch)."""
    _need_cuda(q_in, k_in, q_taps, k_taps, q_norm, k_norm, state, token_req, q_start, slots, out_loc, k_cache, v_cache)
    T, Cq, Ck = q_in.shape[0], q_in.shape[1], k_in.shape[1]
    stride = _rows_view(q_in, Cq, "q")
    assert _rows_view(k_in, Ck, "k") == stride and q_in.dtype == k_in.dtype
    item = q_in.element_size()
    q_off = 0
    k_off = (k_in.data_ptr() - q_in.data_ptr()) // item
    taps = q_taps.shape[0]
    assert q_taps.shape == (taps, Cq) and k_taps.shape == (taps, Ck) and q_taps.dtype == torch.float32 and k_taps.dtype == torch.float32
    assert q_taps.is_contiguous() and k_taps.is_contiguous()
    assert q_norm.dtype == torch.float32 and k_norm.dtype == torch.float32 and q_norm.numel() == Cq and k_norm.numel() == Ck
    assert state.dtype == q_in.dtype and state.is_contiguous() and tuple(state.shape[1:]) == (max(taps - 1, 0), Cq + Ck)
    if k_cache is not None:
        assert k_cache.dtype == q_in.dtype and v_cache.dtype == q_in.dtype and out_loc is not None and out_loc.numel() == T
    q_out = torch.empty((T, Cq), dtype=q_in.dtype, device=q_in.device)
    B = q_start.numel() - 1
    code = _mix_lib().msgl_conv_norm_kvwrite(_ptr(q_in), stride, q_off, k_off, Cq, Ck, head_dim, n_kv, taps, _ptr(q_taps), _ptr(k_taps),
                                             _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(state), _ptr(token_req), _ptr(q_start),
                                             _ptr(slots), _ptr(out_loc), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), page_size, T, B,
                                             int(bool(one_token)), _dt(q_in), _stream())
    _check(code, f"conv_norm_kvwrite ({taps} taps)")
    global LAUNCHES
    LAUNCHES += int(taps > 1 and not (one_token and T == B))
    return q_out


def window_attention_geometry(n_q: int, n_kv: int) -> Tuple[int, int]:
    """(tokens per query tile, query heads of one kv head per block) of the windowed attention kernel."""
    G = n_q // n_kv
    gh = min(G, WINDOW_ATTENTION_ROWS)
    return WINDOW_ATTENTION_ROWS // gh, gh


def window_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *, q_start: torch.Tensor,
                     kv_len: torch.Tensor, block_table: torch.Tensor, n_kv: int, page_size: int, window: int, keep_first: int,
                     scale: float, q_lens: Optional[Sequence[int]], bias: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """Causal softmax attention over the paged cache in which the query at position i sees key j if i - j < window or
    j < keep_first (window <= 0: every earlier key).  bias: float32 [heads, L], added to the scaled score by distance
    min(i - j, L - 1).  gate: [T, heads] (a view into packed rows): the head's output is multiplied by its sigmoid; out_scale
    multiplies everything.  q [T, heads, d]; out [T, heads * d] (may be a view into packed rows).  q_lens: the requests'
    numbers of tokens as the host knows them (they size the launch), or None when every request brings one token."""
    _need_cuda(q, out, k_cache, v_cache, q_start, kv_len, block_table, bias, gate)
    T, n_q, d = q.shape
    assert q.is_contiguous() and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype and out.dtype == q.dtype
    out_stride = _rows_view(out, n_q * d, "out")
    B = kv_len.numel()
    QT, GH = window_attention_geometry(n_q, n_kv)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.dim() == 2 and bias.shape[0] == n_q and bias.is_contiguous()
    gate_stride = 0
    if gate is not None:
        assert gate.dtype == q.dtype
        gate_stride = _rows_view(gate, n_q, "gate")
    n_tiles = sum(-(-n // QT) for n in q_lens) if q_lens is not None else B
    code = _mix_lib().msgl_window_attention(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0),
        int(q_lens is None), n_tiles,
        _ptr(bias), bias.shape[1] if bias is not None else 0, _ptr(gate), gate_stride, 0, _ptr(out), out_stride, 0,
        B, n_q, n_kv, d, page_size, int(window), int(keep_first), QT, GH, float(scale), float(out_scale), _dt(q), _stream())
    _check(code, f"window_attention (head size {d})")


DECAY_CHUNK = 64                 # tokens per chunk of the chunked form of the decaying linear attention
DECAY_CHUNKED_FROM = 16          # a step whose longest request brings this many tokens takes the chunked form


def head_gate(x: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]) * scale; x [T, heads, d] contiguous, gate [T, heads] and out
    [T, heads * d] views into packed rows."""
    _need_cuda(x, gate, out)
    T, H, d = x.shape
    assert x.is_contiguous() and out.dtype == x.dtype
    gs = 0
    if gate is not None:
        assert gate.dtype == x.dtype
        gs = _rows_view(gate, H, "gate")
    code = _mix_lib().msgl_head_gate(_ptr(x), _ptr(gate), gs, 0, _ptr(out), _rows_view(out, H * d, "out"), 0, H, d, float(scale), T,
                                     _dt(x), _stream())
    _check(code, "head_gate")


def decay_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, heads: int, decay: torch.Tensor, state: torch.Tensor,
                    q_start: torch.Tensor, slots: torch.Tensor, q_lens: Optional[Sequence[int]] = None,
                    workspace=None) -> torch.Tensor:
    """Linear attention with a fixed decay per head over the step's tokens, continued from and written back to `state`
    [slots, heads, dk, dv] float32: S <- decay_h S + k v^T, o = S^T q with q, k, v = silu of the given projections
    ([T, heads * dk], [T, heads * dk], [T, heads * dv]: views into one packed projection).  -> float32 [T, heads * dv].
    q_lens: the requests' numbers of tokens as the host knows them; when the longest has DECAY_CHUNKED_FROM or more, the
    step is computed in chunks of DECAY_CHUNK tokens that run in parallel (the same sums in another order), else, and
    without q_lens, every request's tokens are walked in order.  workspace: a parts.Workspace for the chunks' states."""
    _need_cuda(q, k, v, decay, state, q_start, slots)
    T = q.shape[0]
    dk, dv = q.shape[1] // heads, v.shape[1] // heads
    stride = _rows_view(q, heads * dk, "q")
    assert _rows_view(k, heads * dk, "k") == stride and _rows_view(v, heads * dv, "v") == stride and q.dtype == k.dtype == v.dtype
    item = q.element_size()
    k_off, v_off = (k.data_ptr() - q.data_ptr()) // item, (v.data_ptr() - q.data_ptr()) // item
    assert decay.dtype == torch.float32 and decay.numel() == heads
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dk, dv)
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
    B = q_start.numel() - 1
    if q_lens is not None and max(q_lens, default=0) >= DECAY_CHUNKED_FROM:
        n_chunks = sum(-(-n // DECAY_CHUNK) for n in q_lens)
        numel = n_chunks * heads * dk * dv
        U = workspace.get("decay_chunk_states", numel, torch.float32) if workspace is not None else \
            torch.empty(numel, dtype=torch.float32, device=q.device)
        code = _mix_lib().msgl_decay_attention_chunked(_ptr(q), stride, 0, k_off, v_off, heads, dk, dv, _ptr(decay), _ptr(state),
                                                       _ptr(q_start), _ptr(slots), _ptr(out), _ptr(U), n_chunks, B, _dt(q), _stream())
        _check(code, f"decay_attention in chunks (key size {dk})")
        global LAUNCHES
        LAUNCHES += 2
        return out
    code = _mix_lib().msgl_decay_attention(_ptr(q), stride, 0, k_off, v_off, heads, dk, dv, _ptr(decay), _ptr(state), _ptr(q_start),
                                           _ptr(slots), _ptr(out), B, _dt(q), _stream())
    _check(code, f"decay_attention (key size {dk})")
    return out


def rms_gate(x: torch.Tensor, weight: torch.Tensor, eps: float, gate: Optional[torch.Tensor], out: torch.Tensor, scale: float = 1.0) -> None:
    """out = x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate) * scale; x float32 [T, N] contiguous, weight float32 [N],
    gate and out [T, N] views into packed rows of the activation type."""
    _need_cuda(x, weight, gate, out)
    T, N = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32 and weight.numel() == N
    gs = _rows_view(gate, N, "gate") if gate is not None else 0
    if gate is not None:
        assert gate.dtype == out.dtype
    code = _mix_lib().msgl_rms_gate(_ptr(x), N, _ptr(weight), float(eps), _ptr(gate), gs, 0, _ptr(out), _rows_view(out, N, "out"), 0,
                                    float(scale), T, _dt(out), _stream())
    _check(code, "rms_gate")


def gated_act(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor, act: int) -> None:
    """out = act(gate) * up, act = ACT_SILU, ACT_GELU_TANH (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) or ACT_SIGMOID;
    all three [T, I] views into packed rows, gate and up in the same rows."""
    _need_cuda(gate, up, out)
    T, I = gate.shape
    stride = _rows_view(gate, I, "gate")
    assert _rows_view(up, I, "up") == stride and gate.dtype == up.dtype == out.dtype
    up_off = (up.data_ptr() - gate.data_ptr()) // gate.element_size()
    code = _mix_lib().msgl_gated_act(_ptr(gate), stride, 0, up_off, _ptr(out), _rows_view(out, I, "out"), 0, I, int(act), T, _dt(gate),
                                     _stream())
    _check(code, "gated_act")


def scaled_embedding(ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """ids int32 [T], table [V, H] -> float32 [T, H] = float(table[ids]) * scale."""
    _need_cuda(ids, table)
    T, (V, H) = ids.numel(), table.shape
    assert ids.dtype == torch.int32 and table.is_contiguous()
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(_mix_lib().msgl_scaled_embedding(_ptr(ids), _ptr(table), _ptr(out), T, H, V, float(scale), _dt(table), _stream()),
           "scaled_embedding")
    return out


def postnorm_residual(a: torch.Tensor, weight: torch.Tensor, eps: float, scale: float, residual: torch.Tensor, *,
                      next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                      out_dtype: torch.dtype = torch.bfloat16) -> Optional[torch.Tensor]:
    """residual += scale * rmsnorm(a) * weight in float32, in place (a sublayer's output that is normed before it joins the
    stream); with `next_weight` also -> rmsnorm(residual) * next_weight in `out_dtype`, the next sublayer's input, from the same
    pass over the row.  a: [T, H] float32 or `out_dtype`; weights float32 [H]."""
    _need_cuda(a, weight, residual, next_weight)
    T, H = a.shape
    assert a.is_contiguous() and a.dtype in (torch.float32, out_dtype)
    assert residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape == a.shape
    assert weight.dtype == torch.float32 and weight.numel() == H
    y = None
    if next_weight is not None:
        assert next_weight.dtype == torch.float32 and next_weight.numel() == H
        y = torch.empty((T, H), dtype=out_dtype, device=a.device)
    code = _mix_lib().msgl_postnorm_residual(_ptr(a), int(a.dtype == torch.float32), _ptr(weight), float(eps), float(scale),
                                             _ptr(residual), _ptr(next_weight), float(next_eps), _ptr(y), T, H, _DT[out_dtype], _stream())
    _check(code, "postnorm_residual")
    return y


def latent_prep(proj: torch.Tensor, *, dq_off: int, q_rank: int, dkv_off: int, kv_rank: int, rot_dim: int, rot_dims: int,
                dq_norm: Optional[torch.Tensor], dkv_norm: torch.Tensor, eps: float, freq: Optional[torch.Tensor], mag: float,
                positions: torch.Tensor, out_loc: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                page_size: int) -> Optional[torch.Tensor]:
    """What a token of a latent attention leaves in the cache, and its query latent.  proj [T, .] holds the query's
    down-projection (q_rank columns at dq_off; q_rank = 0: none) and the key/value down-projection (kv_rank + rot_dim columns
    at dkv_off).  The cache row of a token (`cache` [pages, 1, page, kv_rank + rot_dim] at token slot out_loc) gets the RMS-normed
    latent followed by the last rot_dim columns, whose first rot_dims are rotated by position * freq (pairs i, i + rot_dims / 2;
    cos and sin times `mag`).  -> the RMS-normed query latent [T, q_rank], or None."""
    _need_cuda(proj, dq_norm, dkv_norm, freq, positions, out_loc, cache)
    T = proj.shape[0]
    assert proj.dim() == 2 and proj.stride(1) == 1 and dkv_off + kv_rank + rot_dim <= proj.shape[1]
    assert dkv_norm.dtype == torch.float32 and dkv_norm.numel() == kv_rank
    assert positions.dtype == torch.int32 and positions.numel() == T
    cq = None
    if q_rank:
        assert dq_norm is not None and dq_norm.dtype == torch.float32 and dq_norm.numel() == q_rank and dq_off + q_rank <= proj.shape[1]
        cq = torch.empty((T, q_rank), dtype=proj.dtype, device=proj.device)
    if rot_dims:
        assert freq is not None and freq.dtype == torch.float32 and freq.numel() == rot_dims // 2
    if cache is not None:
        assert cache.dtype == proj.dtype and cache.is_contiguous() and cache.shape[1] == 1 and cache.shape[3] == kv_rank + rot_dim
        assert out_loc is not None and out_loc.dtype == torch.int32 and out_loc.numel() == T
    code = _mix_lib().msgl_latent_prep(_ptr(proj), proj.stride(0), dq_off, dkv_off, q_rank, kv_rank, rot_dim, rot_dims, _ptr(dq_norm),
                                       _ptr(dkv_norm), float(eps), _ptr(freq), float(mag), _ptr(positions), _ptr(out_loc), _ptr(cq),
                                       _ptr(cache), page_size, T, _dt(proj), _stream())
    _check(code, "latent_prep")
    return cq


def rope_heads(src: torch.Tensor, src_off: int, dst: torch.Tensor, dst_off: int, *, rot_dim: int, rot_dims: int,
               freq: torch.Tensor, mag: float, positions: torch.Tensor) -> None:
    """dst[t, h, dst_off : dst_off + rot_dim] = the part src[t, h, src_off : src_off + rot_dim] of every head with its first
    rot_dims elements rotated by position * freq (pairs i, i + rot_dims / 2; cos and sin times `mag`).  src [T, heads, a] may be
    a view with a row stride of its own, dst [T, heads, b] is contiguous."""
    _need_cuda(src, dst, freq, positions)
    T, heads, sh = src.shape
    assert dst.is_contiguous() and dst.shape[:2] == src.shape[:2] and dst.dtype == src.dtype
    assert src.stride(2) == 1 and src.stride(1) == sh
    assert freq.dtype == torch.float32 and freq.numel() == rot_dims // 2 and positions.dtype == torch.int32
    code = _mix_lib().msgl_rope_heads(_ptr(src), src.stride(0), sh, src_off, _ptr(dst), dst.shape[2], dst_off, heads, rot_dim, rot_dims,
                                      _ptr(freq), float(mag), _ptr(positions), T, _dt(src), _stream())
    _check(code, "rope_heads")


def gate_mul(gate: torch.Tensor, x: torch.Tensor, out: torch.Tensor, act: int) -> None:
    """out = act(gate) * x with act = ACT_SIGMOID or ACT_SILU; [T, N] views into rows of their own strides."""
    _need_cuda(gate, x, out)
    T, N = x.shape
    assert gate.dtype == x.dtype == out.dtype
    code = _mix_lib().msgl_gate_mul(_ptr(gate), _rows_view(gate, N, "gate"), _ptr(x), _rows_view(x, N, "x"), _ptr(out),
                                    _rows_view(out, N, "out"), N, int(act), T, _dt(x), _stream())
    _check(code, "gate_mul")


GATED_DECAY_CHUNKED_FROM = 32    # a step whose longest request brings this many tokens takes the chunked form


def gated_decay_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias: torch.Tensor, *, heads: int,
                          tau: float, q_scale: float, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
                          q_lens: Optional[Sequence[int]] = None, workspace=None) -> torch.Tensor:
    """Linear attention whose decay comes from the input, per token and key channel, continued from and written back to `state`
    [slots, heads, dk, dv] float32: alpha = sigmoid(z + z_bias)^(1 / tau), S <- diag(alpha) S + k v^T, o = S^T (q * q_scale).
    q, k [T, heads * dk] and v [T, heads * dv] are views into one packed projection; z float32 [T, heads * dk] contiguous,
    z_bias float32 [heads * dk].  -> float32 [T, heads * dv].  q_lens: the requests' numbers of tokens as the host knows them
    (None: every request is walked token by token); when the longest has GATED_DECAY_CHUNKED_FROM or more, the step is computed
    in chunks of DECAY_CHUNK tokens that run in parallel (the same sums in another order).  workspace: a parts.Workspace for the
    chunks' scratch."""
    _need_cuda(q, k, v, z, z_bias, state, q_start, slots)
    T = q.shape[0]
    dk, dv = q.shape[1] // heads, v.shape[1] // heads
    stride = _rows_view(q, heads * dk, "q")
    assert _rows_view(k, heads * dk, "k") == stride and _rows_view(v, heads * dv, "v") == stride and q.dtype == k.dtype == v.dtype
    item = q.element_size()
    k_off, v_off = (k.data_ptr() - q.data_ptr()) // item, (v.data_ptr() - q.data_ptr()) // item
    assert z.dtype == torch.float32 and z.is_contiguous() and tuple(z.shape) == (T, heads * dk)
    assert z_bias.dtype == torch.float32 and z_bias.numel() == heads * dk
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dk, dv)
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
    B = q_start.numel() - 1
    if q_lens is not None and max(q_lens, default=0) >= GATED_DECAY_CHUNKED_FROM:
        n_chunks = sum(-(-n // DECAY_CHUNK) for n in q_lens)
        sizes = (("gated_chunk_states", n_chunks * heads * dk * dv), ("gated_chunk_decays", T * heads * dk),
                 ("gated_chunk_weights", n_chunks * heads * DECAY_CHUNK * DECAY_CHUNK))
        U, bcum, P = (workspace.get(name, n, torch.float32) if workspace is not None else
                      torch.empty(n, dtype=torch.float32, device=q.device) for name, n in sizes)
        code = _mix_lib().msgl_gated_decay_attention_chunked(
            _ptr(q), stride, 0, k_off, v_off, heads, dk, dv, _ptr(z), _ptr(z_bias), float(tau), float(q_scale), _ptr(state),
            _ptr(q_start), _ptr(slots), _ptr(out), _ptr(U), _ptr(bcum), _ptr(P), n_chunks, B, _dt(q), _stream())
        _check(code, f"gated_decay_attention in chunks (key size {dk})")
        global LAUNCHES
        LAUNCHES += 4
        return out
    code = _mix_lib().msgl_gated_decay_attention(_ptr(q), stride, 0, k_off, v_off, heads, dk, dv, _ptr(z), _ptr(z_bias), float(tau),
                                                 float(q_scale), _ptr(state), _ptr(q_start), _ptr(slots), _ptr(out), B, _dt(q), _stream())
    _check(code, f"gated_decay_attention (key size {dk})")
    return out


def group_rms_gate(x: torch.Tensor, heads: int, weight: torch.Tensor, eps: float, gate: Optional[torch.Tensor], out: torch.Tensor,
                   act: int = ACT_SILU, scale: float = 1.0) -> None:
    """out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * weight * act(gate[t, h, :]) * scale: an RMS norm over every
    head of a row with one weight [d] for all heads.  x float32 [T, heads * d] contiguous; gate and out [T, heads * d] views
    into packed rows of the activation type; act = ACT_SILU or ACT_SIGMOID."""
    _need_cuda(x, weight, gate, out)
    T, N = x.shape
    d = N // heads
    assert x.dtype == torch.float32 and x.is_contiguous() and N == heads * d and weight.dtype == torch.float32 and weight.numel() == d
    gs = 0
    if gate is not None:
        assert gate.dtype == out.dtype
        gs = _rows_view(gate, N, "gate")
    code = _mix_lib().msgl_group_rms_gate(_ptr(x), heads, d, _ptr(weight), float(eps), _ptr(gate), gs, _ptr(out),
                                          _rows_view(out, N, "out"), float(scale), int(act), T, _dt(out), _stream())
    _check(code, "group_rms_gate")


# ---------------------------------------------------------------------------------------
# sigmoid attention, gated recurrences, state-space scan, routed experts (csrc/mixers_gated.cu)
# ---------------------------------------------------------------------------------------
_gated = None
ACT_RELU2, ACT_RELU = 3, 4
SIGMOID_ATTENTION_ROWS = 8          # (token, head) rows of a block of the sigmoid attention kernel
SIGMOID_ATTENTION_MAX_HEAD_DIM = 512
MINGRU_CHUNK = 32                   # tokens of a chunk when a long portion's recurrence runs in chunks side by side
SIGMOID_ATTENTION_MMA_ROWS = 64     # rows of a block of the tensor-core kernel
SIGMOID_ATTENTION_MMA_MAX_HEAD_DIM = 128
SIGMOID_ATTENTION_SPLIT_KEYS = 256  # keys of a piece when a one-token step cuts a request's keys over several blocks
SSM_MAX_STATE = 512
SSM_CHUNK = 64                      # tokens of a chunk when a long portion's state-space recurrence runs in chunks side by side
SSM_CHUNKED_FROM = 128              # the longest request's tokens from which a step runs in chunks
SSM_CHUNK_MAX_STATE = 256           # state sizes whose chunk tiles fit shared memory
ROUTE_MAX_EXPERTS, ROUTE_MAX_GROUPS = 1024, 64
EXPERTS_FEW_PAIRS = 64              # up to this many (token, choice) pairs the experts' products stream the weights


def _gated_lib():
    global _gated
    if _gated is None:
        lib = _build.gated_mixers_library()
        lib.msgl_embed_positions.argtypes = [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
        lib.msgl_headnorm_kvwrite.argtypes = [c_void_p, c_ll] + [c_int] * 7 + [c_void_p, c_void_p, c_float, c_float, c_int] + \
            [c_void_p] * 5 + [c_int, c_int, c_int, c_void_p]
        lib.msgl_sigmoid_attention.argtypes = [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_ll, c_void_p] + \
            [c_int] * 11 + [c_float, c_int, c_void_p]
        lib.msgl_sigmoid_attention_mma.argtypes = [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_ll, c_void_p] + \
            [c_int] * 9 + [c_float, c_void_p]
        lib.msgl_mingru.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int] + [c_void_p] * 6 + [c_ll, c_float, c_int, c_int, c_void_p]
        lib.msgl_mingru_chunked.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int] + [c_void_p] * 6 + [c_ll, c_float, c_int, c_int, c_int,
                                            c_void_p, c_void_p, c_int, c_void_p]
        lib.msgl_pair_norm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int, c_int, c_void_p]
        lib.msgl_causal_conv_act.argtypes = [c_void_p, c_ll, c_int, c_int, c_int] + [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_ssm_scan.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_int] + [c_void_p] * 7 + [c_int, c_int, c_void_p]
        lib.msgl_ssm_scan_chunked.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_int] + [c_void_p] * 7 + \
            [c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
        lib.msgl_gate_group_norm.argtypes = [c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_ll, c_void_p, c_ll, c_float, c_int,
                                             c_int, c_void_p]
        lib.msgl_unary_act.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_float, c_int, c_int, c_void_p]
        lib.msgl_route.argtypes = [c_void_p, c_ll, c_void_p, c_void_p] + [c_int] * 5 + [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                   c_void_p, c_void_p]
        lib.msgl_experts_few.argtypes = [c_void_p, c_ll] + [c_void_p] * 4 + [c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_int,
                                                                            c_float, c_void_p, c_void_p, c_void_p]
        lib.msgl_clamped_glu.argtypes = [c_void_p, c_ll, c_int, c_float, c_void_p, c_int, c_int, c_void_p]
        lib.msgl_expert_order.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]
        lib.msgl_expert_gather.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p]
        lib.msgl_expert_combine.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p,
                                            c_void_p]
        _gated = lib
    return _gated


def _col_off(view: torch.Tensor, base: torch.Tensor) -> int:
    """Column at which `view` starts inside the packed rows that `base` starts."""
    return (view.data_ptr() - base.data_ptr()) // base.element_size()


def embed_positions(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, places: torch.Tensor, scale: float) -> torch.Tensor:
    """ids, positions int32 [T]; table [V, H], places [P, H] -> float32 [T, H] = float(table[ids]) * scale + float(places[positions])."""
    _need_cuda(ids, positions, table, places)
    T, (V, H) = ids.numel(), table.shape
    assert ids.dtype == torch.int32 and positions.dtype == torch.int32 and table.is_contiguous() and places.is_contiguous()
    assert places.shape[1] == H and places.dtype == table.dtype
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(_gated_lib().msgl_embed_positions(_ptr(ids), _ptr(positions), _ptr(table), _ptr(places), _ptr(out), T, H, V, places.shape[0],
                                             float(scale), _dt(table), _stream()), "embed_positions")
    return out


def headnorm_kvwrite(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor, *, n_q: int, n_kv: int, q_weight: torch.Tensor,
                     k_weight: torch.Tensor, eps: float, temp_coef: float, temp_every: int, positions: torch.Tensor,
                     out_loc: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                     page_size: int) -> torch.Tensor:
    """q_in [T, n_q * d], k_in [T, n_kv * d], v_in [T, n_kv * dv]: views into one packed projection.  Every head of q and of k is
    RMS-normed by itself with one weight [d] for all heads (float32); q is then multiplied by 1 + temp_coef * ln(floor((position +
    1) / temp_every) + 1) (temp_coef 0: not).  The normed k goes to `k_cache` [pages, n_kv, page, d], v as it is to `v_cache`
    [pages, n_kv, page, dv] at token slots `out_loc`; the q rows come back as [T, n_q, d]."""
    _need_cuda(q_in, k_in, v_in, q_weight, k_weight, positions, out_loc, k_cache, v_cache)
    T = q_in.shape[0]
    d, dv = q_in.shape[1] // n_q, v_in.shape[1] // n_kv
    stride = _rows_view(q_in, n_q * d, "q")
    assert _rows_view(k_in, n_kv * d, "k") == stride and _rows_view(v_in, n_kv * dv, "v") == stride and q_in.dtype == k_in.dtype == v_in.dtype
    assert q_weight.dtype == torch.float32 and k_weight.dtype == torch.float32 and q_weight.numel() == d and k_weight.numel() == d
    assert positions.dtype == torch.int32 and positions.numel() >= T
    if k_cache is not None:
        assert k_cache.dtype == q_in.dtype and v_cache.dtype == q_in.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (n_kv, page_size, d) and tuple(v_cache.shape[1:]) == (n_kv, page_size, dv)
        assert out_loc is not None and out_loc.dtype == torch.int32 and out_loc.numel() >= T
    else:
        out_loc = None
    q_out = torch.empty((T, n_q, d), dtype=q_in.dtype, device=q_in.device)
    code = _gated_lib().msgl_headnorm_kvwrite(_ptr(q_in), stride, 0, _col_off(k_in, q_in), _col_off(v_in, q_in), n_q, n_kv, d, dv,
                                              _ptr(q_weight), _ptr(k_weight), float(eps), float(temp_coef), int(temp_every),
                                              _ptr(positions), _ptr(out_loc), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), page_size, T,
                                              _dt(q_in), _stream())
    _check(code, "headnorm_kvwrite")
    return q_out


def sigmoid_attention_geometry(n_q: int, n_kv: int, tensor_cores: bool = False) -> Tuple[int, int]:
    """(tokens per query tile, query heads of one kv head per block) of the sigmoid attention kernels."""
    G = n_q // n_kv
    rows = SIGMOID_ATTENTION_MMA_ROWS if tensor_cores else SIGMOID_ATTENTION_ROWS
    gh = min(G, rows)
    return rows // gh, gh


def sigmoid_attention_on_tensor_cores(dtype: torch.dtype, d: int, dv: int) -> bool:
    """Whether the tensor-core kernel takes these rows: bfloat16, head sizes in steps of 8 up to 128."""
    return dtype == torch.bfloat16 and d % 8 == 0 and dv % 8 == 0 and max(d, dv) <= SIGMOID_ATTENTION_MMA_MAX_HEAD_DIM


def sigmoid_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *, q_start: torch.Tensor,
                      kv_len: torch.Tensor, block_table: torch.Tensor, n_kv: int, page_size: int, scale: float, bias: torch.Tensor,
                      q_lens: Optional[Sequence[int]], workspace=None, tensor_cores: Optional[bool] = None) -> None:
    """Causal attention over the paged cache whose weight of key j for the query at position i is sigmoid(q . k * scale +
    bias[head][min(i - j, L - 1)]), each key by itself (nothing is normed over the keys).  q [T, heads, d]; K cache [pages, n_kv,
    page, d], V cache [pages, n_kv, page, dv]; bias float32 [heads, L]; out [T, heads * dv] (may be a view into packed rows).
    q_lens: the requests' numbers of tokens as the host knows them (they size the launch), or None when every request brings one
    token: the keys are then cut into pieces of SIGMOID_ATTENTION_SPLIT_KEYS for as many blocks as the block table's width asks
    for, whose sums are added in order (workspace: a parts.Workspace for the pieces).  tensor_cores: None = the bfloat16 kernel
    with mma products where it takes the sizes (`sigmoid_attention_on_tensor_cores`), the float32 one elsewhere; False = the float32
    arithmetic kernel in any case."""
    _need_cuda(q, out, k_cache, v_cache, q_start, kv_len, block_table, bias)
    T, n_q, d = q.shape
    dv = v_cache.shape[3]
    assert q.is_contiguous() and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype and out.dtype == q.dtype
    out_stride = _rows_view(out, n_q * dv, "out")
    B = kv_len.numel()
    if tensor_cores is None:
        tensor_cores = sigmoid_attention_on_tensor_cores(q.dtype, d, dv) and out_stride % 2 == 0 and out.data_ptr() % 4 == 0
    QT, GH = sigmoid_attention_geometry(n_q, n_kv, tensor_cores)
    assert bias.dtype == torch.float32 and bias.dim() == 2 and bias.shape[0] == n_q and bias.is_contiguous()
    uniform = q_lens is None
    n_tiles = B if uniform else sum(-(-n // QT) for n in q_lens)
    splits, part = 1, None
    if uniform:
        splits = max(1, -(-(block_table.shape[1] * page_size) // SIGMOID_ATTENTION_SPLIT_KEYS))
        if splits > 1:
            numel = splits * T * n_q * dv
            part = workspace.get("sigmoid_attention_pieces", numel, torch.float32) if workspace is not None else \
                torch.empty(numel, dtype=torch.float32, device=q.device)
    if tensor_cores:
        code = _gated_lib().msgl_sigmoid_attention_mma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0), int(uniform),
            n_tiles, _ptr(bias), bias.shape[1], _ptr(out), out_stride, _ptr(part), splits, SIGMOID_ATTENTION_SPLIT_KEYS, T, B, n_q,
            n_kv, d, dv, page_size, float(scale), _stream())
    else:
        code = _gated_lib().msgl_sigmoid_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0), int(uniform),
            n_tiles, _ptr(bias), bias.shape[1], _ptr(out), out_stride, _ptr(part), splits, SIGMOID_ATTENTION_SPLIT_KEYS, T, B, n_q, n_kv,
            d, dv, page_size, QT, GH, float(scale), _dt(q), _stream())
    _check(code, f"sigmoid_attention (head sizes {d}, {dv})")
    if splits > 1:
        global LAUNCHES
        LAUNCHES += 1


def mingru(z: torch.Tensor, x: torch.Tensor, g: torch.Tensor, z_bias: torch.Tensor, x_bias: torch.Tensor, *, state: torch.Tensor,
           q_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, scale: float = 1.0, q_lens: Optional[Sequence[int]] = None,
           workspace=None) -> None:
    """A gated recurrence per channel over the step's tokens, continued from and written back to `state` [slots, W] float32:
    zz = sigmoid(z + z_bias), a = x + x_bias, c = a + 1/2 where a >= 0 and sigmoid(a) below, S <- (1 - zz) S + zz c;
    out = S * silu(g) * scale.  z, x, g [T, W]: views into one packed projection; out [T, W] (may be a view).  q_lens: the
    requests' numbers of tokens as the host knows them; with a request of 2 * MINGRU_CHUNK tokens or more the tokens run in chunks
    side by side (same sums in float32, another order), else one by one."""
    _need_cuda(z, x, g, z_bias, x_bias, state, q_start, slots, out)
    T, W = z.shape
    stride = _rows_view(z, W, "z")
    assert _rows_view(x, W, "x") == stride and _rows_view(g, W, "g") == stride and z.dtype == x.dtype == g.dtype == out.dtype
    assert z_bias.dtype == torch.float32 and x_bias.dtype == torch.float32 and z_bias.numel() == W and x_bias.numel() == W
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (W,)
    B = q_start.numel() - 1
    if q_lens is not None and max(q_lens, default=0) >= 2 * MINGRU_CHUNK:
        L = MINGRU_CHUNK
        n_chunks = sum(-(-n // L) for n in q_lens)
        numel = (2 * n_chunks + B) * W
        buf = workspace.get("mingru_chunks", numel, torch.float32) if workspace is not None else \
            torch.empty(numel, dtype=torch.float32, device=z.device)
        code = _gated_lib().msgl_mingru_chunked(_ptr(z), stride, 0, _col_off(x, z), _col_off(g, z), W, _ptr(z_bias), _ptr(x_bias), _ptr(state),
                                                _ptr(q_start), _ptr(slots), _ptr(out), _rows_view(out, W, "out"), float(scale), B, L,
                                                n_chunks, _ptr(buf), _ptr(buf[2 * n_chunks * W:]), _dt(z), _stream())
        _check(code, "mingru (chunks)")
        global LAUNCHES
        LAUNCHES += 1
        return
    code = _gated_lib().msgl_mingru(_ptr(z), stride, 0, _col_off(x, z), _col_off(g, z), W, _ptr(z_bias), _ptr(x_bias), _ptr(state),
                                    _ptr(q_start), _ptr(slots), _ptr(out), _rows_view(out, W, "out"), float(scale), B, _dt(z), _stream())
    _check(code, "mingru")


def pair_norm(a: torch.Tensor, b: torch.Tensor, a_weight: torch.Tensor, b_weight: torch.Tensor, eps: float, scale: float) -> torch.Tensor:
    """-> float32 [T, H] = scale * (a / rms(a) * a_weight + b / rms(b) * b_weight), each row normed by itself; a, b [T, H] float32 or
    bfloat16 (both alike), weights float32 [H]."""
    _need_cuda(a, b, a_weight, b_weight)
    T, H = a.shape
    assert a.is_contiguous() and b.is_contiguous() and a.shape == b.shape and a.dtype == b.dtype
    assert a_weight.dtype == torch.float32 and b_weight.dtype == torch.float32 and a_weight.numel() == H and b_weight.numel() == H
    _dt(a)
    out = torch.empty((T, H), dtype=torch.float32, device=a.device)
    _check(_gated_lib().msgl_pair_norm(_ptr(a), _ptr(b), int(a.dtype == torch.float32), _ptr(a_weight), _ptr(b_weight), float(eps),
                                       float(scale), _ptr(out), T, H, _stream()), "pair_norm")
    return out


def causal_conv_act(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], *, state: Optional[torch.Tensor],
                    token_req: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, act: int = ACT_SILU) -> torch.Tensor:
    """Short causal convolution over time on every channel of x [T, C] (a view into packed rows) with taps [K, C] (float32, the
    oldest input's tap first) and bias [C], then silu (act = ACT_SILU) or nothing (act < 0); continued from `state` [slots, K - 1,
    C] (the request's last inputs, oldest first), which the call brings up to date.  -> [T, C] contiguous."""
    _need_cuda(x, taps, bias, state, token_req, q_start, slots)
    T, C = x.shape
    K = taps.shape[0]
    assert taps.shape == (K, C) and taps.dtype == torch.float32 and taps.is_contiguous()
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == C
    if K > 1:
        assert state is not None and state.dtype == x.dtype and state.is_contiguous() and tuple(state.shape[1:]) == (K - 1, C)
    out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    B = q_start.numel() - 1
    code = _gated_lib().msgl_causal_conv_act(_ptr(x), _rows_view(x, C, "x"), 0, C, K, _ptr(taps), _ptr(bias), _ptr(state), _ptr(token_req),
                                             _ptr(q_start), _ptr(slots), _ptr(out), 0 if act == ACT_SILU else -1, T, B, _dt(x), _stream())
    _check(code, f"causal_conv_act ({K} taps)")
    if K > 1:
        global LAUNCHES
        LAUNCHES += 1
    return out


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, *, heads: int, groups: int, state_size: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             skip: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
             q_lens: Optional[Sequence[int]] = None, workspace=None) -> torch.Tensor:
    """State-space recurrence per head over the step's tokens, continued from and written back to `state` [slots, heads, N, P]
    float32: step = softplus(dt + dt_bias), S <- exp(-exp(a_log) step) S + step B x^T, y = S^T C + skip x, with head h on group
    h // (heads / groups).  xbc [T, heads * P + 2 groups * N] contiguous = x | B | C; dt [T, heads] a view into packed rows.
    -> float32 [T, heads * P].  q_lens: the requests' numbers of tokens as the host knows them; when the longest has
    SSM_CHUNKED_FROM or more (and the state size is at most SSM_CHUNK_MAX_STATE) the step is computed in chunks of SSM_CHUNK tokens
    that run side by side (the same sums in float32, another order), else, and without q_lens, every request's tokens are walked in
    order.  workspace: a parts.Workspace for the chunks' states."""
    _need_cuda(xbc, dt, dt_bias, a_log, skip, state, q_start, slots)
    T = xbc.shape[0]
    N = state_size
    P = (xbc.shape[1] - 2 * groups * N) // heads
    assert xbc.is_contiguous() and xbc.shape[1] == heads * P + 2 * groups * N and dt.dtype == xbc.dtype
    for w in (dt_bias, a_log, skip):
        assert w.dtype == torch.float32 and w.numel() == heads
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, N, P)
    y = torch.empty((T, heads * P), dtype=torch.float32, device=xbc.device)
    B = q_start.numel() - 1
    if q_lens is not None and max(q_lens, default=0) >= SSM_CHUNKED_FROM and N <= SSM_CHUNK_MAX_STATE:
        n_chunks = sum(-(-n // SSM_CHUNK) for n in q_lens)
        numel = n_chunks * heads * (N * P + 1)
        buf = workspace.get("ssm_chunk_states", numel, torch.float32) if workspace is not None else \
            torch.empty(numel, dtype=torch.float32, device=xbc.device)
        code = _gated_lib().msgl_ssm_scan_chunked(_ptr(xbc), heads, groups, N, P, _ptr(dt), _rows_view(dt, heads, "dt"), 0, _ptr(dt_bias),
                                                  _ptr(a_log), _ptr(skip), _ptr(state), _ptr(q_start), _ptr(slots), _ptr(y), B, n_chunks,
                                                  _ptr(buf), _ptr(buf[n_chunks * heads * N * P:]), _dt(xbc), _stream())
        _check(code, f"ssm_scan in chunks (state size {N})")
        global LAUNCHES
        LAUNCHES += 2
        return y
    code = _gated_lib().msgl_ssm_scan(_ptr(xbc), heads, groups, N, P, _ptr(dt), _rows_view(dt, heads, "dt"), 0, _ptr(dt_bias), _ptr(a_log),
                                      _ptr(skip), _ptr(state), _ptr(q_start), _ptr(slots), _ptr(y), B, _dt(xbc), _stream())
    _check(code, f"ssm_scan (state size {N})")
    return y


def gate_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, parts: int, eps: float, out: torch.Tensor,
                    scale: float = 1.0) -> None:
    """out = v / rms(v) * weight * scale with v = y * silu(gate) and the root mean square taken over each of `parts` equal parts of
    the row by itself (the gate comes before the norm).  y float32 [T, N] contiguous; gate and out [T, N] views into packed rows of
    the activation type; weight float32 [N]."""
    _need_cuda(y, gate, weight, out)
    T, N = y.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and weight.dtype == torch.float32 and weight.numel() == N and gate.dtype == out.dtype
    code = _gated_lib().msgl_gate_group_norm(_ptr(y), N, int(parts), _ptr(weight), float(eps), _ptr(gate), _rows_view(gate, N, "gate"),
                                             _ptr(out), _rows_view(out, N, "out"), float(scale), T, _dt(out), _stream())
    _check(code, "gate_group_norm")


def unary_act(x: torch.Tensor, act: int, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x) * scale, element by element; act = ACT_SILU, ACT_GELU_TANH, ACT_SIGMOID, ACT_RELU2 (relu(x)^2) or ACT_RELU."""
    _need_cuda(x, out)
    T, N = x.shape
    if out is None:
        out = torch.empty((T, N), dtype=x.dtype, device=x.device)
    assert out.dtype == x.dtype
    code = _gated_lib().msgl_unary_act(_ptr(x), _rows_view(x, N, "x"), _ptr(out), _rows_view(out, N, "out"), N, int(act), float(scale), T,
                                       _dt(x), _stream())
    _check(code, "unary_act")
    return out


def route(h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], *, n_groups: int, keep: int,
          top: int, softmax: bool = False, gate_row: Optional[torch.Tensor] = None):
    """The experts a token uses and their weights.  Scores s = sigmoid(router h) with float32 sums; the choice goes by s +
    correction among the experts of the `keep` best of `n_groups` equal groups of neighbouring experts (a group counts by the sum
    of its two largest choice scores), the `top` largest win; the weights are the winners' s over their sum.
    h [T, H], router [E, H] -> (int32 [T, top], float32 [T, top]).
    softmax: the logits router h themselves are what the choice goes by (the largest win, the lower index at a tie), and the
    weights are the softmax over the chosen logits only.  gate_row [H]: one more row that is no expert; the call then returns
    a third tensor, float32 [T] = sigmoid(gate_row . h)."""
    _need_cuda(h, router, correction, gate_row)
    T, H = h.shape
    E = router.shape[0]
    assert router.shape == (E, H) and router.is_contiguous() and router.dtype == h.dtype
    if correction is not None:
        assert correction.dtype == torch.float32 and correction.numel() == E
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=h.device)
    gate_out = None
    if gate_row is not None:
        assert gate_row.dtype == h.dtype and gate_row.numel() == H and gate_row.is_contiguous()
        gate_out = torch.empty(T, dtype=torch.float32, device=h.device)
    code = _gated_lib().msgl_route(_ptr(h), _rows_view(h, H, "h"), _ptr(router), _ptr(correction), H, E, int(n_groups), int(keep),
                                   int(top), _ptr(idx), _ptr(wts), T, _dt(h), int(bool(softmax)), _ptr(gate_row), _ptr(gate_out), _stream())
    _check(code, f"route ({E} experts)")
    if softmax or gate_row is not None:
        return idx, wts, gate_out
    return idx, wts


def experts_few(h: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor,
                scale: float = 1.0, limit: float = 0.0, extra: Optional[torch.Tensor] = None,
                extra_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """-> float32 [T, H] = scale * sum_k wts[t, k] * down[e] (silu(gate[e] h_t) * (up[e] h_t)), e = idx[t, k], with the chosen
    experts' rows read straight from the stacked weights gate_up [E, 2, F, H] (an expert's gate, then its up) and down [E, H, F]:
    for a few tokens.  limit > 0: the activation is g * sigmoid(1.702 g) * (u + 1) with g = min(gate, limit) and
    u = clamp(up, -limit, limit).  extra float32 [T, H] (a shared expert's output) is added inside the sum, times
    extra_gate float32 [T] where given."""
    _need_cuda(h, gate_up, down, idx, wts, extra, extra_gate)
    if extra is not None:
        assert extra.dtype == torch.float32 and extra.is_contiguous() and tuple(extra.shape) == tuple(h.shape)
        assert extra_gate is None or (extra_gate.dtype == torch.float32 and extra_gate.numel() == h.shape[0])
    T, H = h.shape
    E, _, F, _ = gate_up.shape
    top = idx.shape[1]
    assert gate_up.shape == (E, 2, F, H) and down.shape == (E, H, F)
    assert gate_up.is_contiguous() and down.is_contiguous() and gate_up.dtype == down.dtype == h.dtype
    assert idx.dtype == torch.int32 and wts.dtype == torch.float32 and idx.is_contiguous() and wts.is_contiguous()
    act = torch.empty((T * top, F), dtype=h.dtype, device=h.device)
    out = torch.empty((T, H), dtype=torch.float32, device=h.device)
    code = _gated_lib().msgl_experts_few(_ptr(h), _rows_view(h, H, "h"), _ptr(gate_up), _ptr(down), _ptr(idx), _ptr(wts), top, H, F,
                                         _ptr(act), float(scale), _ptr(out), T, _dt(h), float(limit), _ptr(extra),
                                         _ptr(extra_gate) if extra is not None else None, _stream())
    _check(code, "experts_few")
    global LAUNCHES
    LAUNCHES += 1
    return out


def expert_order(idx: torch.Tensor, n_experts: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """idx int32 [T, top] -> (counts int32 [E]: pairs per expert; place int32 [T * top]: row of every (token, choice) pair when the
    pairs are put in the order of their experts, pairs of one expert in their own order)."""
    _need_cuda(idx)
    assert idx.dtype == torch.int32 and idx.is_contiguous()
    counts = torch.empty(n_experts, dtype=torch.int32, device=idx.device)
    place = torch.empty(idx.numel(), dtype=torch.int32, device=idx.device)
    _check(_gated_lib().msgl_expert_order(_ptr(idx), idx.numel(), n_experts, _ptr(counts), _ptr(place), _stream()), "expert_order")
    global LAUNCHES
    LAUNCHES += 1
    return counts, place


def expert_gather(h: torch.Tensor, place: torch.Tensor, top: int) -> torch.Tensor:
    """rows[place[t * top + k]] = h[t]: every token's row once per expert it uses, in expert order."""
    _need_cuda(h, place)
    T, H = h.shape
    rows = torch.empty((T * top, H), dtype=h.dtype, device=h.device)
    _check(_gated_lib().msgl_expert_gather(_ptr(h), _rows_view(h, H, "h"), _ptr(place), top, H, _ptr(rows), T * top, _dt(h), _stream()),
           "expert_gather")
    return rows


def clamped_glu(gate_up: torch.Tensor, limit: float) -> torch.Tensor:
    """[T, 2F] (gate first) -> [T, F] = g * sigmoid(1.702 g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    _need_cuda(gate_up)
    T, F = gate_up.shape[0], gate_up.shape[1] // 2
    assert gate_up.dim() == 2 and gate_up.shape[1] == 2 * F
    out = torch.empty((T, F), dtype=gate_up.dtype, device=gate_up.device)
    _check(_gated_lib().msgl_clamped_glu(_ptr(gate_up), _rows_view(gate_up, 2 * F, "gate_up"), F, float(limit), _ptr(out), T, _dt(gate_up),
                                         _stream()), "clamped_glu")
    return out


def expert_combine(y: torch.Tensor, place: torch.Tensor, wts: torch.Tensor, scale: float = 1.0, extra: Optional[torch.Tensor] = None,
                   extra_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """-> float32 [T, H] = scale * (sum_k wts[t, k] * y[place[t * top + k]] + extra_gate[t] * extra[t]); y [T * top, H] float32 or
    bfloat16; extra float32 [T, H] and extra_gate float32 [T] are optional (no gate: the extra term counts fully)."""
    _need_cuda(y, place, wts, extra, extra_gate)
    if extra is not None:
        assert extra.dtype == torch.float32 and extra.is_contiguous() and extra.shape[1] == y.shape[1]
        assert extra_gate is None or (extra_gate.dtype == torch.float32 and extra_gate.numel() == wts.shape[0])
    T, top = wts.shape
    H = y.shape[1]
    assert y.is_contiguous() and y.shape[0] == T * top and wts.dtype == torch.float32 and wts.is_contiguous()
    _dt(y)
    out = torch.empty((T, H), dtype=torch.float32, device=y.device)
    _check(_gated_lib().msgl_expert_combine(_ptr(y), int(y.dtype == torch.float32), _ptr(place), _ptr(wts), top, H, float(scale), _ptr(out),
                                            T, _ptr(extra), _ptr(extra_gate) if extra is not None else None, _stream()), "expert_combine")
    return out


# ---------------------------------------------------------------------------------------
# attention with a sink, the gated delta rule, scaled sums and the per-layer token input (csrc/mixers_delta.cu)
# ---------------------------------------------------------------------------------------
_delta = None
SINK_ATTENTION_ROWS = 8             # (token, head) rows of a block of the attention kernel with a sink
SINK_ATTENTION_MAX_HEAD_DIM = 512
SINK_ATTENTION_SPLIT_KEYS = 256     # keys of a piece when a one-token step cuts a request's keys over several blocks
DELTA_RULE_MAX_KEY_DIM = 512


def _delta_lib():
    global _delta
    if _delta is None:
        lib = _build.delta_mixers_library()
        lib.msgl_scaled_add_norm.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.msgl_rotary_angles.argtypes = [c_void_p, c_void_p, ctypes.c_double, c_void_p, c_int, c_int, c_void_p]
        lib.msgl_sink_qkv_prep.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_void_p, c_ll, c_float] + [c_void_p] * 4 + [c_int] * 7 + [c_void_p]
        lib.msgl_sink_attention.argtypes = [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p, c_void_p, c_ll, c_void_p, c_void_p] + \
            [c_int] * 12 + [c_float, c_float, c_int, c_void_p]
        lib.msgl_sink_attention_mma.argtypes = [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p, c_void_p, c_ll, c_void_p, c_void_p] + \
            [c_int] * 10 + [c_float, c_float, c_void_p]
        lib.msgl_delta_rule.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_int] + [c_void_p] * 7 + [c_int] * 7 + [c_void_p]
        lib.msgl_delta_rule_scratch.argtypes = [c_int] * 4
        lib.msgl_delta_rule_scratch.restype = c_ll
        lib.msgl_side_gate_mul.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
        _delta = lib
    return _delta


def scaled_add_norm(x: torch.Tensor, scale: torch.Tensor, residual: torch.Tensor, *, weight: Optional[torch.Tensor] = None,
                    eps: float = 0.0, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """residual += x * scale in float32, in place (scale: float32 [H], one factor per column).  With `weight` (float32 [H])
    -> rmsnorm(residual) * weight in `out_dtype`, from the same pass; without it -> residual itself in `out_dtype`, or nothing
    when `out_dtype` is None.  x [T, H] float32 or bfloat16."""
    _need_cuda(x, scale, residual, weight)
    T, H = x.shape
    assert x.is_contiguous() and x.dtype in (torch.float32, torch.bfloat16)
    assert residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape == x.shape
    assert scale.dtype == torch.float32 and scale.numel() == H and (weight is None or (weight.dtype == torch.float32 and weight.numel() == H))
    y = torch.empty((T, H), dtype=out_dtype, device=x.device) if out_dtype is not None else None
    assert weight is None or y is not None
    code = _delta_lib().msgl_scaled_add_norm(_ptr(x), int(x.dtype == torch.float32), _ptr(scale), _ptr(residual), _ptr(weight), float(eps),
                                             _ptr(y), _DT[out_dtype] if out_dtype is not None else 0, T, H, _stream())
    _check(code, "scaled_add_norm")
    return y


def rotary_angles(positions: torch.Tensor, freq: torch.Tensor, magnitude: float, T: int) -> torch.Tensor:
    """positions int32 [>= T], freq float64 [n] -> float32 [T, 2n] = magnitude * (cos | sin)(position * freq), the product and the
    circular functions in double precision."""
    _need_cuda(positions, freq)
    assert positions.dtype == torch.int32 and positions.numel() >= T and freq.dtype == torch.float64 and freq.is_contiguous()
    n = freq.numel()
    out = torch.empty((T, 2 * n), dtype=torch.float32, device=freq.device)
    _check(_delta_lib().msgl_rotary_angles(_ptr(positions), _ptr(freq), float(magnitude), _ptr(out), T, n, _stream()), "rotary_angles")
    return out


def sink_qkv_prep(proj: torch.Tensor, *, n_q: int, n_kv: int, d: int, dv: int, angles: Optional[torch.Tensor],
                  v_first: Optional[torch.Tensor], lam: float, out_loc: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                  v_cache: Optional[torch.Tensor], page_size: int) -> torch.Tensor:
    """proj [T, >= n_q * d + n_kv * d + n_kv * dv] packed rows [q | k | v | ...].  The first angles.shape[1] elements of every q and
    k head turn in halves (element i against i + rot / 2) by `angles` float32 [T, rot] = cos | sin of the tokens' positions; v
    becomes (1 - lam) v + lam v_first where `v_first` [T, n_kv * dv] (a view into packed rows) is given; k goes to `k_cache`
    [pages, n_kv, page, d] and v to `v_cache` [pages, n_kv, page, dv] at token slots `out_loc`; the q rows come back as [T, n_q, d]."""
    _need_cuda(proj, angles, v_first, out_loc, k_cache, v_cache)
    T = proj.shape[0]
    width = (n_q + n_kv) * d + n_kv * dv
    stride = _rows_view(proj, proj.shape[1], "proj")
    assert proj.shape[1] >= width
    rot = 0
    if angles is not None:
        rot = angles.shape[1]
        assert angles.dtype == torch.float32 and angles.is_contiguous() and angles.shape[0] >= T
    vf_stride = 0
    if v_first is not None:
        assert v_first.dtype == proj.dtype and v_first.shape == (T, n_kv * dv)
        vf_stride = _rows_view(v_first, n_kv * dv, "v_first")
    if k_cache is not None:
        assert k_cache.dtype == proj.dtype and v_cache.dtype == proj.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (n_kv, page_size, d) and tuple(v_cache.shape[1:]) == (n_kv, page_size, dv)
        assert out_loc is not None and out_loc.dtype == torch.int32 and out_loc.numel() >= T
    q_out = torch.empty((T, n_q, d), dtype=proj.dtype, device=proj.device)
    code = _delta_lib().msgl_sink_qkv_prep(_ptr(proj), stride, _ptr(angles), rot, _ptr(v_first), vf_stride, float(lam), _ptr(out_loc),
                                           _ptr(q_out), _ptr(k_cache), _ptr(v_cache), page_size, n_q, n_kv, d, dv, T, _dt(proj), _stream())
    _check(code, "sink_qkv_prep")
    return q_out


SINK_ATTENTION_MMA_ROWS = 64        # rows of a block of the tensor-core kernel
SINK_ATTENTION_MMA_MAX_HEAD_DIM = 128


def sink_attention_geometry(n_q: int, n_kv: int, tensor_cores: bool = False) -> Tuple[int, int]:
    """(tokens per query tile, query heads of one kv head per block) of the attention kernels with a sink."""
    rows = SINK_ATTENTION_MMA_ROWS if tensor_cores else SINK_ATTENTION_ROWS
    gh = min(n_q // n_kv, rows)
    return rows // gh, gh


def sink_attention_on_tensor_cores(dtype: torch.dtype, d: int, dv: int) -> bool:
    """Whether the tensor-core kernel takes these rows: bfloat16, head sizes in steps of 8 up to 128."""
    return dtype == torch.bfloat16 and d % 8 == 0 and dv % 8 == 0 and max(d, dv) <= SINK_ATTENTION_MMA_MAX_HEAD_DIM


def sink_attention_splits(table_width: int, page_size: int, window: int) -> int:
    """Pieces a one-token step cuts a request's keys into: as many as the block table's width asks for, or as a window touches."""
    splits = max(1, -(-(table_width * page_size) // SINK_ATTENTION_SPLIT_KEYS))
    if window > 0:
        splits = min(splits, (window - 1) // SINK_ATTENTION_SPLIT_KEYS + 2)
    return splits


def sink_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *, q_start: torch.Tensor,
                   kv_len: torch.Tensor, block_table: torch.Tensor, n_kv: int, page_size: int, scale: float, softcap: float,
                   window: int, sink: torch.Tensor, q_lens: Optional[Sequence[int]], workspace=None,
                   tensor_cores: Optional[bool] = None) -> None:
    """Causal softmax attention over the paged cache: the query at position i sees the keys j <= i with i - j < window (window 0:
    all), score = q . k * scale, capped as softcap * tanh(score / softcap) where softcap > 0, and every softmax's denominator
    holds exp(sink[head]) besides the seen keys' terms.  q [T, heads, d]; K cache [pages, n_kv, page, d], V cache [pages, n_kv,
    page, dv]; sink float32 [heads]; out [T, heads * dv].  q_lens: the requests' numbers of tokens as the host knows them (they
    size the launch), or None when every request brings one token: the keys are then cut into pieces of
    SINK_ATTENTION_SPLIT_KEYS for blocks of their own, joined in order by a second kernel (workspace: a parts.Workspace for
    the pieces).  tensor_cores: None = the bfloat16 kernel with mma products where it takes the sizes
    (`sink_attention_on_tensor_cores`), the float32-arithmetic one elsewhere; False = the float32-arithmetic kernel in any case."""
    _need_cuda(q, out, k_cache, v_cache, q_start, kv_len, block_table, sink)
    T, n_q, d = q.shape
    dv = v_cache.shape[3]
    assert q.is_contiguous() and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype and out.dtype == q.dtype
    assert sink.dtype == torch.float32 and sink.numel() == n_q
    out_stride = _rows_view(out, n_q * dv, "out")
    B = kv_len.numel()
    if tensor_cores is None:
        tensor_cores = sink_attention_on_tensor_cores(q.dtype, d, dv) and out_stride % 2 == 0 and out.data_ptr() % 4 == 0
    QT, GH = sink_attention_geometry(n_q, n_kv, tensor_cores)
    uniform = q_lens is None
    n_tiles = B if uniform else sum(-(-n // QT) for n in q_lens)
    splits, part_o, part_ml = 1, None, None
    if uniform:
        splits = sink_attention_splits(block_table.shape[1], page_size, int(window))
        if splits > 1:
            rows = splits * T * n_q
            if workspace is not None:
                part_o, part_ml = workspace.get("sink_attention_o", rows * dv, torch.float32), workspace.get("sink_attention_ml", rows * 2, torch.float32)
            else:
                part_o = torch.empty(rows * dv, dtype=torch.float32, device=q.device)
                part_ml = torch.empty(rows * 2, dtype=torch.float32, device=q.device)
    if tensor_cores:
        code = _delta_lib().msgl_sink_attention_mma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0), int(uniform),
            n_tiles, _ptr(sink), _ptr(out), out_stride, _ptr(part_o), _ptr(part_ml), splits, SINK_ATTENTION_SPLIT_KEYS, T, B, n_q, n_kv, d,
            dv, page_size, int(window), float(scale), float(softcap), _stream())
    else:
        code = _delta_lib().msgl_sink_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0), int(uniform),
            n_tiles, _ptr(sink), _ptr(out), out_stride, _ptr(part_o), _ptr(part_ml), splits, SINK_ATTENTION_SPLIT_KEYS, T, B, n_q, n_kv, d,
            dv, page_size, QT, GH, int(window), float(scale), float(softcap), _dt(q), _stream())
    _check(code, f"sink_attention (head sizes {d}, {dv})")
    if splits > 1:
        global LAUNCHES
        LAUNCHES += 1


def delta_rule(qkv: torch.Tensor, a: torch.Tensor, b: torch.Tensor, *, heads: int, kv_heads: int, key_dim: int, value_dim: int,
               a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
               q_lens: Optional[Sequence[int]] = None, workspace=None) -> torch.Tensor:
    """The gated delta rule over the step's tokens, continued from and written back to `state` [slots, heads, key_dim, value_dim]
    float32.  qkv [T, 2 * kv_heads * key_dim + heads * value_dim] contiguous (q | k | v as the convolution left them); a, b
    [T, heads]: views into one packed projection (decay and write-strength pre-activations).  Per head: unit-length q (times
    key_dim^-1/2) and k, beta = sigmoid(b), g = exp(-exp(a_log) softplus(a + dt_bias)), S <- g S, u = beta (v - S^T k),
    S <- S + k u^T, o = S^T q.  -> float32 [T, heads * value_dim]."""
    _need_cuda(qkv, a, b, a_log, dt_bias, state, q_start, slots)
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == 2 * kv_heads * key_dim + heads * value_dim
    assert a.dtype == qkv.dtype and b.dtype == qkv.dtype and a.shape == (T, heads) and b.shape == (T, heads)
    stride = _rows_view(a, heads, "a")
    assert _rows_view(b, heads, "b") == stride
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, key_dim, value_dim)
    assert a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32 and a_log.numel() == heads and dt_bias.numel() == heads
    out = torch.empty((T, heads * value_dim), dtype=torch.float32, device=qkv.device)
    B = q_start.numel() - 1
    # what does not depend on the state (unit q and k, beta, g) is made for all tokens at once by a kernel of its own
    numel = int(_delta_lib().msgl_delta_rule_scratch(T, heads, kv_heads, key_dim))
    scratch = workspace.get("delta_rule_prep", numel, torch.float32) if workspace is not None else \
        torch.empty(numel, dtype=torch.float32, device=qkv.device)
    code = _delta_lib().msgl_delta_rule(_ptr(qkv), _ptr(a), stride, 0, _col_off(b, a), _ptr(a_log), _ptr(dt_bias), _ptr(state), _ptr(q_start),
                                        _ptr(slots), _ptr(out), _ptr(scratch), heads, kv_heads, key_dim, value_dim, T, B, _dt(qkv), _stream())
    _check(code, f"delta_rule (key size {key_dim})")
    global LAUNCHES
    LAUNCHES += 1
    return out


def side_gate_mul(gate: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, offset: int) -> torch.Tensor:
    """gate [T, dim], table [V, columns], ids int32 [T] -> [T, dim] = gelu_tanh(gate) * table[ids][offset : offset + dim]."""
    _need_cuda(gate, table, ids)
    T, dim = gate.shape
    assert table.dtype == gate.dtype and table.is_contiguous() and ids.dtype == torch.int32 and ids.numel() >= T
    out = torch.empty((T, dim), dtype=gate.dtype, device=gate.device)
    code = _delta_lib().msgl_side_gate_mul(_ptr(gate), _rows_view(gate, dim, "gate"), _ptr(table), table.shape[1], int(offset), _ptr(ids),
                                           table.shape[0], _ptr(out), dim, T, _dt(gate), _stream())
    _check(code, "side_gate_mul")
    return out


# ---------------------------------------------------------------------------------------
# the whole decode step in one persistent kernel (csrc/decode_step.cu)
# ---------------------------------------------------------------------------------------
# Off unless MSGL_FUSED_DECODE=1: measured on B200 at Qwen3-8B's sizes the one-kernel step takes 4.2 / 5.4 ms at batch 1 / 8
# (context 4,096) against 3.4 / 4.2 ms kernel by kernel (see profiles/decode_step_kernel_b1_b8.md for where the time goes).
USE_FUSED_DECODE = os.environ.get("MSGL_FUSED_DECODE", "0") == "1"
FUSED_DECODE_MAX_TOKENS = 8
STATUS_WORD_DECODE_STEP = 3


class DsLayer(ctypes.Structure):
    """One run of a layer for the decode-step kernel; mirrors `struct DsLayer`."""
    _fields_ = [("w_qkv", c_void_p), ("b_qkv", c_void_p), ("w_o", c_void_p), ("w_gu", c_void_p), ("w_down", c_void_p),
                ("norm_in", c_void_p), ("norm_post", c_void_p), ("q_norm", c_void_p), ("k_norm", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("eps_in", c_float), ("eps_post", c_float), ("eps_qk", c_float),
                ("norm_f32", c_int), ("qk_norm_f32", c_int), ("pad_", c_int)]


class DsStep(ctypes.Structure):
    """Arguments of one decode step; mirrors `struct DsStep`."""
    _fields_ = [("layers", c_void_p), ("n_layers", c_int), ("M", c_int),
                ("H", c_int), ("n_q", c_int), ("n_kv", c_int), ("I", c_int), ("V", c_int),
                ("page_size", c_int), ("page_shift", c_int), ("bt_stride", c_int), ("max_split", c_int),
                ("scale", c_float),
                ("rope", c_void_p), ("rot", c_int), ("max_pos", c_int),
                ("ids", c_void_p), ("positions", c_void_p), ("kv_len", c_void_p), ("block_table", c_void_p),
                ("out_loc", c_void_p), ("nsplit", c_void_p),
                ("embed", c_void_p), ("final_norm", c_void_p), ("final_f32", c_int), ("eps_final", c_float),
                ("lm_head", c_void_p),
                ("res", c_void_p), ("xn", c_void_p), ("ssq", c_void_p), ("qkv", c_void_p), ("attn", c_void_p), ("act", c_void_p),
                ("part_o", c_void_p), ("part_ml", c_void_p), ("tickets", c_void_p), ("logits", c_void_p),
                ("bar", c_void_p), ("status", c_void_p)]


_decode_libs = {}


def _decode_lib(head_dim: int):
    lib = _decode_libs.get(head_dim)
    if lib is None:
        lib = _build.decode_step_library(head_dim)
        lib.msgl_decode_step_blocks.argtypes = [c_int] * 6
        lib.msgl_decode_step_blocks.restype = c_int
        lib.msgl_decode_step.argtypes = [ctypes.POINTER(DsStep), c_void_p]
        if lib.msgl_decode_step_layer_bytes() != ctypes.sizeof(DsLayer) or lib.msgl_decode_step_struct_bytes() != ctypes.sizeof(DsStep):
            raise KernelError("decode_step: the argument structures of the library and of ops.py differ")
        _decode_libs[head_dim] = lib
    return lib


def decode_step_blocks(tokens: int, hidden: int, n_q: int, n_kv: int, head_dim: int, intermediate: int, vocab: int) -> int:
    """Blocks the decode-step kernel runs with for these sizes on the current device; 0: it does not take them
    (the caller then runs the step kernel by kernel).  Not inside a stream capture the first time."""
    if not USE_FUSED_DECODE or head_dim % 32 or head_dim < 32 or head_dim > 128:      # beyond 128 the accumulators spill
        return 0
    return int(_decode_lib(head_dim).msgl_decode_step_blocks(tokens, hidden, n_q, n_kv, intermediate, vocab))


def decode_step(step: DsStep, head_dim: int) -> None:
    """Launch the decode-step kernel on the current stream."""
    code = _decode_lib(head_dim).msgl_decode_step(ctypes.byref(step), _stream())
    _check(code, f"decode_step (head size {head_dim})")
