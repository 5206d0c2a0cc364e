"""The hand-written sm_100a kernels as Python functions over torch tensors.

Each function checks on the host what the kernel relies on (device, dtype,
contiguity, shapes, alignment), then passes raw pointers and the current CUDA
stream to the C entry point.  There is no other implementation behind these
names: without a CUDA device, nvcc or the compiled library they raise.

`linear_bf16` is the one place where a library matrix product stands (cuBLAS
through torch, for more than 64 rows), as the reference's engine uses a library
for its products (`engine/backend.go:265-267`, `mlxc/mlxc.go:655`).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..csrc import build

PAGE = 64                      # tokens per cache page (JANIS_PAGE in the CUDA sources)
GEMV_MAX_ROWS = 64             # what the skinny kernel accepts
GEMV_FAST_ROWS = 16            # up to here it beats the library product (above, each warp re-reads too much of x)
TC05_MAX_ROWS = 64             # rows the tcgen05 skinny product takes
EPI_NONE, EPI_GATED_GELU, EPI_SOFTCAP, EPI_GATED_SILU = 0, 1, 2, 3
GATE_GROUP = 8                 # fused gate/up rows alternate in groups of 8
ACT_GELU_TANH, ACT_SILU = 0, 1

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


def _need_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("janis_b200 runs on a CUDA device only: torch.cuda.is_available() is False "
                          "and there is no CPU implementation")


_core = None
_attn: dict[int, ctypes.CDLL] = {}


def core():
    global _core
    if _core is None:
        _need_cuda()
        lib = build.core_library()
        P, I, F = c_void_p, c_int, c_float
        lib.janis_embed.argtypes = [P, P, I, P, I, I, I, F, P]
        lib.janis_rmsnorm.argtypes = [P, I, P, P, P, I, I, I, F, P]
        lib.janis_add_rmsnorm.argtypes = [P, P, I, I, c_longlong, P, F, P, F, P, I, I, I, P]
        lib.janis_gated_act.argtypes = [P, P, I, I, I, I, I, P]
        lib.janis_softcap.argtypes = [P, c_longlong, F, P]
        lib.janis_scale_values.argtypes = [P, c_longlong, F, P]
        lib.janis_bias_act.argtypes = [P, P, I, I, I, I, F, F, P]
        lib.janis_rope_store.argtypes = [P, I, P, P, P, P, P, I, I, I, I, I, I, P, P, P, I, I, I, P]
        lib.janis_kv_store.argtypes = [P, I, P, P, P, P, I, I, I, I, I, P, P, P, I, I, P]
        lib.janis_gemm_f32.argtypes = [P, P, P, I, I, I, F, P]
        lib.janis_gemv_bf16.argtypes = [P, P, P, I, I, I, I, I, F, I, P]
        lib.janis_gemv_bf16_bias_act.argtypes = [P, P, P, I, I, I, P, I, F, F, P]
        lib.janis_gemv_rope_store.argtypes = [P, P, P, I, I, P, P, P, P, P, I, I, I, I, P, P, P, I, I, P]
        lib.janis_gemm_tc05.argtypes = [P, P, P, I, I, I, I, I, F, I, P]
        lib.janis_tc05_timeouts.restype = I
        lib.janis_tc05_timeouts_async.argtypes = [P, P]
        lib.janis_tc05_set_stages.argtypes = [I]
        lib.janis_tc05_set_stages.restype = None
        lib.janis_argmax.argtypes = [P, P, I, I, P]
        lib.janis_sample.argtypes = [P, P, P, I, I, F, F, c_ulonglong, P, P, P]
        lib.janis_set_sample_kernel.argtypes = [I]
        lib.janis_set_sample_kernel.restype = None
        lib.janis_repeat_penalty.argtypes = [P, P, I, I, I, F, P]
        lib.janis_mask_tokens.argtypes = [P, P, I, I, I, P]
        lib.janis_set_overlap.argtypes = [I]
        lib.janis_set_overlap.restype = None
        lib.janis_set_overlap(1 if _overlap else 0)
        _core = lib
    return _core


def attention_lib(head_dim: int):
    lib = _attn.get(head_dim)
    if lib is None:
        _need_cuda()
        lib = build.attention_library(head_dim)
        P, I, F = c_void_p, c_int, c_float
        lib.janis_attn_head_dim.restype = I
        lib.janis_attn_decode_scratch.argtypes = [I, I, I]
        lib.janis_attn_decode_scratch.restype = c_longlong
        lib.janis_attn_prefill.argtypes = [P, P, I, P, P, P, P, I, I, I, I, I, I, F, F, I, P, P, P, P, P, I, I, P]
        lib.janis_attn_decode.argtypes = [P, P, P, I, P, I, P, P, P, c_longlong, P, I, I, I, I, F, F, I, I, I, I, P]
        lib.janis_attn_prefill_mma.argtypes = [P, P, I, P, P, I, I, P, I, I, I, I, I, F, F, I, P, c_longlong,
                                               P, P, P, P, P, I, I, I, P]
        lib.janis_attn_set_prefill_kernel.argtypes = [I]
        lib.janis_attn_set_prefill_kernel.restype = None
        lib.janis_attn_set_prefill_piece.argtypes = [I]
        lib.janis_attn_set_prefill_piece.restype = None
        lib.janis_attn_set_decode_wide.argtypes = [I]
        lib.janis_attn_set_decode_wide.restype = None
        lib.janis_attn_set_prefill_items.argtypes = [I]
        lib.janis_attn_set_prefill_items.restype = None
        lib.janis_attn_prefill_kernels.argtypes = []
        lib.janis_attn_prefill_kernels.restype = I
        lib.janis_attn_prefill_piece.argtypes = [I, I, I, I, I, I]
        lib.janis_attn_prefill_piece.restype = I
        lib.janis_attn_tc05_timeouts.restype = I
        lib.janis_attn_timeouts_async.argtypes = [P, P]
        lib.janis_attn_prefill_scratch.argtypes = [I, I]
        lib.janis_attn_prefill_scratch.restype = c_longlong
        lib.janis_attn_prefill_tile.restype = I
        lib.janis_attn_set_decode_kernel.argtypes = [I]
        lib.janis_attn_set_decode_kernel.restype = None
        lib.janis_attn_decode_stages.argtypes = [c_longlong]
        lib.janis_attn_decode_stages.restype = I
        lib.janis_attn_set_decode_stages.argtypes = [I]
        lib.janis_attn_set_decode_stages.restype = None
        lib.janis_attn_wait_timeouts.restype = I
        lib.janis_attn_wait_probe.argtypes = [I, P, P]
        lib.janis_attn_set_overlap.argtypes = [I]
        lib.janis_attn_set_overlap.restype = None
        lib.janis_attn_set_overlap(1 if _overlap else 0)
        if lib.janis_attn_head_dim() != head_dim:
            raise KernelError(f"attention library for head size {head_dim} reports {lib.janis_attn_head_dim()}")
        _attn[head_dim] = lib
    return lib


_mixers = None


def mixers():
    """The library of the mixers whose sizes are run-time numbers (compiled when a model first needs it)."""
    global _mixers
    if _mixers is None:
        _need_cuda()
        lib = build.mixers_library()
        P, I, F = c_void_p, c_int, c_float
        lib.janis_qkv_rotate_store.argtypes = [P, I, I, P, P, P, P, I, P, I, I, I, I, I, I, P, P, P, I, P]
        lib.janis_talk_attention.argtypes = [P, I, I, P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, I, I, I, P, c_longlong, I, F, P, I, I, P, c_longlong, I, P]
        lib.janis_talk_attention_set_kernel.argtypes = [I]
        lib.janis_talk_attention_set_kernel.restype = None
        lib.janis_talk_attention_rows_floats.argtypes = [I, I, I, I, I, I, I]
        lib.janis_talk_attention_rows_floats.restype = c_longlong
        lib.janis_talk_attention_rows.argtypes = [P, I, I, P, P, P, P, P, P, I, P, P, I, I, I, I, I, F, I, I, I, F, P, I, P, c_longlong, I, P]
        lib.janis_gla_scan.argtypes = [P, I, I, I, I, I, P, P, P, I, P, P, P, P, P, P, I, I, I, I, F, F, P]
        lib.janis_head_norm_gate.argtypes = [P, P, I, I, I, P, F, P, I, I, I, I, I, P]
        lib.janis_mlstm_scan.argtypes = [P, I, I, I, I, I, P, P, F, P, I, P, P, P, P, P, P, P, P, I, I, I, I, F, P]
        lib.janis_causal_conv_silu.argtypes = [P, I, I, I, I, I, P, P, P, P, P, P, P, P, I, I, I, P, I, P]
        lib.janis_conv_state_update.argtypes = [P, I, I, I, I, I, P, P, P, P, P, I, P]
        lib.janis_qkv_conv_norm_store.argtypes = [P, I, I, I, I, I, I, I, I, P, P, P, P, I, F, P, P, P, P, P, P, P, P, P, P, I, P]
        lib.janis_latent_rotate_store.argtypes = [P, I, I, I, P, I, I, I, I, I, I, I, I, P, F, P, F, P, P, P, P, P, P, I, P]
        lib.janis_qk_rotate_norm_store.argtypes = [P, I, I, I, I, I, I, I, I, P, I, F, P, P, P, P, P, P, I, P]
        lib.janis_head_linear.argtypes = [P, I, I, I, I, P, P, I, I, I, I, I, I, I, P]
        lib.janis_group_norm.argtypes = [P, P, I, P, F, P, F, I, P, I, I, I, P]
        lib.janis_round_rows.argtypes = [P, P, ctypes.c_size_t, P]
        lib.janis_selective_scan.argtypes = [P, I, I, I, P, I, I, P, P, I, P, I, I, I, P, P, I, I, P, P, P, P, I, P, P, I, I, I, I, I, P, P]
        lib.janis_selective_scan_set_lanes.argtypes = [I]
        lib.janis_selective_scan_set_lanes.restype = None
        lib.janis_selective_scan_set_form.argtypes = [I]
        lib.janis_selective_scan_set_form.restype = None
        lib.janis_gate_group_norm.argtypes = [P, P, I, I, I, P, F, I, P, I, I, P]
        lib.janis_dyt_norm.argtypes = [P, P, I, P, F, P, P, P, I, I, I, P]
        lib.janis_rmsnorm_accumulate.argtypes = [P, I, P, F, F, P, I, I, I, P]
        lib.janis_sigmoid_gate.argtypes = [P, P, I, I, I, I, I, I, P]
        lib.janis_moe_route.argtypes = [P, P, I, I, I, I, I, F, I, P, I, I, P]
        lib.janis_moe_expert_act.argtypes = [P, I, P, I, I, F, I, F, F, P, I, I, F, P]
        lib.janis_moe_identity_add.argtypes = [P, P, I, P, I, I, I, I, P]
        lib.janis_hc_spread.argtypes = [P, P, I, I, I, P]
        lib.janis_hc_read_norm.argtypes = [P, P, P, P, F, P, I, I, I, I, P]
        lib.janis_hc_update.argtypes = [P, P, I, P, P, P, P, F, P, I, I, I, P]
        lib.janis_mixers_set_overlap.argtypes = [I]
        lib.janis_mixers_set_overlap.restype = None
        lib.janis_mixers_set_overlap(1 if _overlap else 0)
        _mixers = lib
    return _mixers


_overlap = os.environ.get("JANIS_OVERLAP", "1") != "0"


def set_overlap(on: bool) -> None:
    """Whether a kernel's CTAs may arrive while the kernel before it in the stream still runs
    (programmatic dependent launch; every kernel waits for its predecessor before it touches
    anything but weights and the step's tables).  Results are the same either way."""
    global _overlap
    _overlap = bool(on)
    if _core is not None:
        _core.janis_set_overlap(1 if _overlap else 0)
    for lib in _attn.values():
        lib.janis_attn_set_overlap(1 if _overlap else 0)
    if _mixers is not None:
        _mixers.janis_mixers_set_overlap(1 if _overlap else 0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  (A prompt step launches some three hundred kernels from Python; building a
    Stream object for each took a fifth of the step's host time.)"""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """How many of this library's kernels have been launched (or recorded into a graph) so far."""
    return _launches


def _check(lib, rc: int, kernels: int = 1) -> None:
    global _launches
    if rc != 0:
        raise KernelError(lib.janis_last_error().decode("utf-8", "replace"))
    _launches += kernels


def _t(x: torch.Tensor, name: str, dtype=None, shape=None) -> int:
    """The address of a tensor an entry point is given, after the checks the C side cannot make: on the device,
    contiguous, of an accepted dtype (one, or a tuple), of the wanted shape (None: any extent)."""
    try:
        if not x.is_cuda:
            raise KernelError(f"{name}: expected a CUDA tensor")
    except AttributeError:
        raise KernelError(f"{name}: expected a CUDA tensor") from None
    if not x.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None:
        xd = x.dtype
        if xd != dtype and not (type(dtype) in (tuple, list) and xd in dtype):
            raise KernelError(f"{name}: dtype {xd} not accepted here (wanted {dtype})")
    if shape is not None:
        xs = x.shape
        bad = len(xs) != len(shape)
        if not bad:
            for want, have in zip(shape, xs):
                if want is not None and want != have:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{name}: shape {tuple(xs)} does not match {tuple(shape)}")
    return x.data_ptr()


_FLOATS = (torch.float32, torch.bfloat16)

# ---------------------------------------------------------------------------
# rows of the residual stream
# ---------------------------------------------------------------------------

def embed(tokens, table, scale: float, out):
    """out[t] = float(table[tokens[t]]) * scale;  tokens int32 [T], table [V, H], out float32 [T, H]."""
    T = tokens.numel()
    V, H = table.shape
    lib = core()
    _check(lib, lib.janis_embed(_t(tokens, "tokens", torch.int32), _t(table, "table", _FLOATS), _DT[table.dtype],
                                _t(out, "out", torch.float32, (T, H)), T, H, V, float(scale), _stream()))
    return out


def rmsnorm(x, weight, eps: float, out, rows=None):
    """out[r] = x[rows[r] or r] / sqrt(mean(x^2) + eps) * weight;  weight float32 holds offset + w."""
    H = x.shape[-1]
    R = out.shape[0]
    if rows is None and x.shape[0] != R:
        raise KernelError(f"rmsnorm: {x.shape[0]} input rows for {R} output rows")
    lib = core()
    _check(lib, lib.janis_rmsnorm(_t(x, "x", _FLOATS, (None, H)), _DT[x.dtype], _t(weight, "weight", torch.float32, (H,)),
                                  _t(rows, "rows", torch.int32, (R,)) if rows is not None else None,
                                  _t(out, "out", _FLOATS, (R, H)), _DT[out.dtype], R, H, float(eps), _stream()))
    return out


def add_rmsnorm(h, res, w_post, eps_post, w_next=None, eps_next=0.0, out=None, n_part=1):
    """h += norm(res; w_post) in place (float32 residual sum; h += res when w_post is None);
    out = norm(h; w_next) when w_next is given.
    `res` is [R, H], or [n_part, R, H] partial results that are added first."""
    R, H = h.shape
    if n_part == 1:
        _t(res, "res", _FLOATS, (R, H))
        stride = 0
    else:
        _t(res, "res", _FLOATS, (n_part, R, H))
        stride = R * H
    lib = core()
    _check(lib, lib.janis_add_rmsnorm(
        _t(h, "h", torch.float32, (R, H)), res.data_ptr(), _DT[res.dtype], n_part, stride,
        _t(w_post, "w_post", torch.float32, (H,)) if w_post is not None else None, float(eps_post),
        _t(w_next, "w_next", torch.float32, (H,)) if w_next is not None else None, float(eps_next),
        _t(out, "out", _FLOATS, (R, H)) if out is not None else None,
        _DT[out.dtype] if out is not None else 0, R, H, _stream()))
    return out


def gated_act(gu, out, act: int = ACT_GELU_TANH, group: int = GATE_GROUP):
    """out[r, j] = act(gate) * up over a fused [R, 2I] product whose columns alternate
    `group` gate columns and `group` up columns."""
    R, I2 = gu.shape
    I = I2 // 2
    lib = core()
    _check(lib, lib.janis_gated_act(_t(gu, "gu", _FLOATS, (R, 2 * I)), _t(out, "out", gu.dtype, (R, I)),
                                    _DT[gu.dtype], R, I, group, act, _stream()))
    return out


ACT_NONE, ACT_XIELU, ACT_GELU, ACT_SILU_PLAIN, ACT_RELU2 = 0, 1, 2, 3, 4


def bias_act(x, bias, act: int = ACT_NONE, a_pos: float = 0.0, a_neg: float = 0.0):
    """x = act(x + bias) in place over [R, N] (bias [N] of x's dtype, or None).  ACT_XIELU takes the two numbers
    a_pos and a_neg: z > 0: a_pos z^2 + z/2; z <= 0: a_neg (e^z - 1 - z) + z/2."""
    R, N = x.shape
    lib = core()
    _check(lib, lib.janis_bias_act(_t(x, "x", _FLOATS, (R, N)), _t(bias, "bias", x.dtype, (N,)) if bias is not None else None,
                                   _DT[x.dtype], R, N, int(act), float(a_pos), float(a_neg), _stream()))
    return x


def rope_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, rot: int, nq: int, nkv: int, hd: int,
               kpool=None, vpool=None, page_table=None, ring_len: int = 0, store: bool = True,
               write_cache: bool = True):
    """Rotate q and k of qkv [T, heads, hd] (heads = q, then k, then v) in place and write k and v into
    the paged cache.

    kpool/vpool: [pages, nkv, PAGE, hd] of one cache line; page_table int32 [slots, pages per sequence].
    With store=False the rows hold q alone and only q is rotated (a layer that reads another layer's
    keys).  With write_cache=False q and k are rotated and nothing is stored (`kv_store` does it later)."""
    T = qkv.shape[0]
    row_heads = nq + 2 * nkv if store else nq
    _t(qkv, "qkv", _FLOATS, (T, row_heads, hd))
    _t(tok_pos, "tok_pos", torch.int32)
    _t(tok_seq, "tok_seq", torch.int32)
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("rope_store: position tables shorter than the step")
    _t(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    stride = 0
    if store and not write_cache:
        lib = core()
        _check(lib, lib.janis_rope_store(qkv.data_ptr(), _DT[qkv.dtype], tok_pos.data_ptr(), tok_seq.data_ptr(), None,
                                         None, inv_freq.data_ptr(), rot, T, nq, nkv, hd, row_heads, None, None, None,
                                         0, 0, 0, _stream()))
        return qkv
    if store:
        n_pages = kpool.shape[0]
        _t(kpool, "kpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
        _t(vpool, "vpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
        _t(page_table, "page_table", torch.int32, (None, None))
        _t(seq_slot, "seq_slot", torch.int32)
        _t(seq_end, "seq_end", torch.int32)
        stride = page_table.shape[1]
    lib = core()
    _check(lib, lib.janis_rope_store(
        qkv.data_ptr(), _DT[qkv.dtype], tok_pos.data_ptr(), tok_seq.data_ptr(),
        seq_slot.data_ptr() if store else None, seq_end.data_ptr() if store else None,
        inv_freq.data_ptr(), rot, T, nq, nkv, hd, row_heads,
        kpool.data_ptr() if store else None, vpool.data_ptr() if store else None,
        page_table.data_ptr() if store else None, stride, ring_len, 0 if store else 1, _stream()))
    return qkv


def kv_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, nq: int, nkv: int, hd: int, kpool, vpool, page_table,
             ring_len: int = 0):
    """Write the keys and values of qkv [T, nq + 2 nkv, hd] into the paged cache line as they stand (the places
    and the rule for rings are rope_store's): the second half of `rope_store(..., write_cache=False)`."""
    T = qkv.shape[0]
    _t(qkv, "qkv", _FLOATS, (T, None, hd))
    if qkv.shape[1] < nq + 2 * nkv:
        raise KernelError("kv_store: the rows of qkv hold no keys and values")
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(vpool, "vpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(page_table, "page_table", torch.int32, (None, None))
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("kv_store: position tables shorter than the step")
    lib = core()
    _check(lib, lib.janis_kv_store(qkv.data_ptr(), _DT[qkv.dtype], _t(tok_pos, "tok_pos", torch.int32),
                                   _t(tok_seq, "tok_seq", torch.int32), _t(seq_slot, "seq_slot", torch.int32),
                                   _t(seq_end, "seq_end", torch.int32), T, nq, nkv, hd, qkv.shape[1], kpool.data_ptr(),
                                   vpool.data_ptr(), page_table.data_ptr(), page_table.shape[1], int(ring_len), _stream()))
    return qkv


# ---------------------------------------------------------------------------
# products
# ---------------------------------------------------------------------------

def gemm_f32(x, w, out, cap: float = 0.0):
    """out[M, N] = x[M, K] w[N, K]^T in true float32 (CUDA cores); optional cap * tanh(v / cap)."""
    M, K = x.shape
    N = w.shape[0]
    lib = core()
    _check(lib, lib.janis_gemm_f32(_t(x, "x", torch.float32, (M, K)), _t(w, "w", torch.float32, (N, K)),
                                   _t(out, "out", torch.float32, (M, N)), M, N, K, float(cap), _stream()))
    return out


def gemv_bf16(x, w, out, epilogue: int = EPI_NONE, cap: float = 0.0, cluster: int = 0):
    """out = x[M<=64, K] w[N, K]^T, bfloat16 operands, float accumulation; out bfloat16 or float32
    [M, N], or [M, N/2] with a gated epilogue (rows of w alternate 8 gate rows and 8 up rows).
    cluster: how many CTAs of a thread-block cluster share the K of a tile (1, 2, 4; 0 = chosen from N, K)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in (EPI_GATED_GELU, EPI_GATED_SILU) else N
    lib = core()
    _check(lib, lib.janis_gemv_bf16(_t(x, "x", torch.bfloat16, (M, K)), _t(w, "w", torch.bfloat16, (N, K)),
                                    _t(out, "out", _FLOATS, (M, n_out)), _DT[out.dtype], M, N, K, epilogue,
                                    float(cap), int(cluster), _stream()))
    return out


def gemv_bf16_bias_act(x, w, out, bias, act: int = 0, a_pos: float = 0.0, a_neg: float = 0.0):
    """out = act(bf16(x w^T) + bias) for up to 64 rows in one kernel: the bits that `gemv_bf16` into bfloat16 followed
    by `bias_act` leaves (bias [N] bfloat16 or None; act and its two numbers as in `bias_act`)."""
    M, K = x.shape
    N = w.shape[0]
    lib = core()
    _check(lib, lib.janis_gemv_bf16_bias_act(_t(x, "x", torch.bfloat16, (M, K)), _t(w, "w", torch.bfloat16, (N, K)),
                                             _t(out, "out", torch.bfloat16, (M, N)), M, N, K,
                                             _t(bias, "bias", torch.bfloat16, (N,)) if bias is not None else None,
                                             int(act), float(a_pos), float(a_neg), _stream()))
    return out


def gemv_rope_store(x, w, qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, nq: int, nkv: int, hd: int,
                    kpool=None, vpool=None, page_table=None, ring_len: int = 0, store: bool = True):
    """The q/k/v projection of up to 16 decode rows with the rotary encoding of the whole head and the cache write
    in its epilogue: what `gemv_bf16(x, w, qkv)` followed by `rope_store(qkv, ...)` leaves in the queries' part
    of qkv [M, heads, hd] and in the cache line, in one kernel (the keys' and values' part of qkv is not written).
    w: [(nq + 2 nkv) hd, K], or [nq hd, K] with store=False (a layer that reads another layer's keys)."""
    M, K = x.shape
    heads = nq + 2 * nkv if store else nq
    _t(x, "x", torch.bfloat16, (M, K))
    _t(w, "w", torch.bfloat16, (heads * hd, K))
    _t(qkv, "qkv", torch.bfloat16, (M, None, hd))
    if qkv.shape[1] < nq:
        raise KernelError("gemv_rope_store: the rows of qkv hold fewer heads than nq")
    _t(tok_pos, "tok_pos", torch.int32)
    _t(tok_seq, "tok_seq", torch.int32)
    if tok_pos.numel() < M or tok_seq.numel() < M:
        raise KernelError("gemv_rope_store: position tables shorter than the step")
    _t(inv_freq, "inv_freq", torch.float32, (hd // 2,))
    stride = 0
    if store:
        n_pages = kpool.shape[0]
        _t(kpool, "kpool", torch.bfloat16, (n_pages, nkv, PAGE, hd))
        _t(vpool, "vpool", torch.bfloat16, (n_pages, nkv, PAGE, hd))
        _t(page_table, "page_table", torch.int32, (None, None))
        _t(seq_slot, "seq_slot", torch.int32)
        _t(seq_end, "seq_end", torch.int32)
        stride = page_table.shape[1]
    lib = core()
    _check(lib, lib.janis_gemv_rope_store(
        x.data_ptr(), w.data_ptr(), qkv.data_ptr(), M, K, tok_pos.data_ptr(), tok_seq.data_ptr(),
        seq_slot.data_ptr() if store else None, seq_end.data_ptr() if store else None, inv_freq.data_ptr(),
        nq, nkv, hd, qkv.shape[1], kpool.data_ptr() if store else None, vpool.data_ptr() if store else None,
        page_table.data_ptr() if store else None, stride, ring_len, _stream()))
    return qkv


def softcap(x, cap: float):
    """x = cap * tanh(x / cap) in place, float32."""
    lib = core()
    _check(lib, lib.janis_softcap(_t(x, "x", torch.float32), x.numel(), float(cap), _stream()))
    return x


def scale_values(x, factor: float):
    """x *= factor in place, float32 (a constant on the logits)."""
    lib = core()
    _check(lib, lib.janis_scale_values(_t(x, "x", torch.float32), x.numel(), float(factor), _stream()))
    return x


def gemm_tc05(x, w, out, epilogue: int = EPI_NONE, cap: float = 0.0, split: int = 0):
    """out = x[M<=64, K] w[N, K]^T on the tcgen05 tensor cores (operands swapped: rows of w fill the 128 TMEM
    lanes, the batch rows are the narrow side), TMA-fed, K split over a cluster when N is small.  Same
    epilogues and output shapes as gemv_bf16.  split: CTAs that share K (1, 2, 4, 8; 0 = chosen from N, K)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in (EPI_GATED_GELU, EPI_GATED_SILU) else N
    lib = core()
    _check(lib, lib.janis_gemm_tc05(_t(x, "x", torch.bfloat16, (M, K)), _t(w, "w", torch.bfloat16, (N, K)),
                                    _t(out, "out", _FLOATS, (M, n_out)), _DT[out.dtype], M, N, K, epilogue,
                                    float(cap), int(split), _stream()))
    return out


def tc05_set_stages(stages: int = 0) -> None:
    """Fix the depth of the tcgen05 product's ring of stages (3 to 9; 0: chosen from the CTAs per SM, the default).
    For tests and tuning."""
    core().janis_tc05_set_stages(int(stages))


def tc05_timeouts() -> int:
    """How often a CTA of gemm_tc05 gave up waiting on a barrier (0 in a healthy run); synchronises."""
    return int(core().janis_tc05_timeouts())


class WaitWatch:
    """Notices when a kernel has given up one of its bounded waits (on a barrier of its copies or of its tensor-core
    products): such a CTA returns without its result, and what the step produced is then worthless.

    `request()` asks every loaded library, in the order of the current stream and without waiting, to copy its
    counters of given-up waits into pinned host memory; `check()`, called once the host has waited for that
    stream anyway (to read the step's tokens), raises `KernelError` if a counter has grown since the last
    check.  Counters of libraries loaded later join at their next request."""

    def __init__(self):
        self._host = torch.zeros(64, dtype=torch.int32).pin_memory()
        self._where: dict[str, int] = {}           # library -> index of its first counter
        self._seen = [0] * 64

    def _slot(self, name: str) -> int:              # two counters a library (core: the tcgen05 product's waits, the clusters' of the skinny products)
        if name not in self._where:
            if 2 * len(self._where) + 2 > 64:
                raise KernelError("too many attention libraries for one watch")
            self._where[name] = 2 * len(self._where)
        return self._where[name]

    def request(self) -> None:
        st, base = _stream(), self._host.data_ptr()
        if _core is not None:
            _check(_core, _core.janis_tc05_timeouts_async(base + 4 * self._slot("core"), st), 0)
        for hd, lib in _attn.items():
            _check(lib, lib.janis_attn_timeouts_async(base + 4 * self._slot(f"attention (head size {hd})"), st), 0)

    def check(self, quiet: bool = False) -> None:
        """Call after the stream of the last `request()` has been waited for (quiet: take note, raise nothing)."""
        now = self._host.tolist()
        grown = [(name, now[at + i] - self._seen[at + i]) for name, at in self._where.items() for i in range(2)
                 if now[at + i] > self._seen[at + i]]
        self._seen = now
        if grown and not quiet:
            what = ", ".join(f"{n} in {name}" for name, n in grown)
            raise KernelError(f"a kernel gave up a bounded wait ({what}): the results of the steps since the last "
                              "check are not to be trusted")


def linear_bf16(x, w, out):
    """out[M, N] = x w^T in bfloat16 with float accumulation: the skinny kernel up to 16 rows (inner sizes that
    are multiples of 8), the library product (cuBLAS) otherwise."""
    M = x.shape[0]
    if M <= GEMV_FAST_ROWS and x.shape[1] % 8 == 0:
        return gemv_bf16(x, w, out)
    _t(x, "x", torch.bfloat16)
    _t(w, "w", torch.bfloat16)
    _t(out, "out", torch.bfloat16, (M, w.shape[0]))
    torch.mm(x, w.t(), out=out)
    return out


def matmul_bf16_to_f32(x, w, out):
    """out[M, N] float32 = x[M, K] w[N, K]^T, bfloat16 operands, the library product (cuBLAS)."""
    _t(x, "x", torch.bfloat16)
    _t(w, "w", torch.bfloat16)
    _t(out, "out", torch.float32, (x.shape[0], w.shape[0]))
    torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    return out


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------

def attn_prefill_scratch_floats(n_tok: int, n_seq: int, nq: int, hd: int, dtype=torch.bfloat16) -> int:
    """Floats of scratch that attn_prefill wants for a step of n_tok tokens in n_seq sequences: a bfloat16
    step with few tiles of queries shares each long tile between up to four CTAs, which meet through the scratch
    (0: nothing is shared).  Without the scratch the step runs unshared."""
    if dtype != torch.bfloat16:
        return 0
    lib = attention_lib(hd)
    bm = lib.janis_attn_prefill_tile()
    return int(lib.janis_attn_prefill_scratch((n_tok + bm - 1) // bm + n_seq, nq))


def _cached_args(name, seq_start, seq_slot, kpool, vpool, page_table, ring_len, dtype, n_seq, nkv, hd):
    """The arguments that say where the keys and values of earlier steps are (all null for a step whose sequences
    start at position 0)."""
    if seq_start is None:
        return (None, None, None, None, None, 0, 0)
    if kpool is None or vpool is None or page_table is None or seq_slot is None:
        raise KernelError(f"{name}: sequences that continue need their slots and the cache line")
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", dtype, (n_pages, nkv, PAGE, hd))
    _t(vpool, "vpool", dtype, (n_pages, nkv, PAGE, hd))
    _t(page_table, "page_table", torch.int32, (None, None))
    _t(seq_start, "seq_start", torch.int32)
    _t(seq_slot, "seq_slot", torch.int32)
    if n_seq is not None and (seq_start.numel() < n_seq or seq_slot.numel() < n_seq):
        raise KernelError(f"{name}: sequence tables shorter than the step")
    return (seq_start.data_ptr(), seq_slot.data_ptr(), kpool.data_ptr(), vpool.data_ptr(), page_table.data_ptr(),
            page_table.shape[1], int(ring_len))


def attn_prefill(qkv, tok_pos, tok_seq, seq_first_row, out, nq: int, nkv: int, hd: int, scale: float, cap: float,
                 window: int, kv_src=None, kv_row_heads=None, kv_k_head0=None, seq_len=None, tensor_cores=True,
                 scratch=None, seq_start=None, seq_slot=None, kpool=None, vpool=None, page_table=None,
                 ring_len: int = 0, host_lens=None):
    """Causal (and windowed when window > 0) attention over packed sequences.
    qkv: [T, nq + 2 nkv, hd], or [T, nq, hd] when keys and values come from `kv_src`, another layer's
    [T, kv_row_heads, hd] rows whose key heads start at head kv_k_head0 (values nkv heads later).
    Without `seq_start` every sequence starts at position 0 and seq_first_row is the row of that position.  With
    `seq_start` (int32 [n_seq], the tokens earlier steps stored) the step continues sequences: tok_pos are absolute
    positions, seq_first_row is the row of a sequence's first token of this step, `seq_len` the lengths after the
    step, and the keys and values of earlier positions are read from the cache line (kpool, vpool, page_table,
    ring_len), which must still hold what those steps left (this step's own keys are stored afterwards).
    `host_lens`: the tokens each sequence brings to this step, if the host knows them (a step replayed from a graph
    with other lengths does not): the grid then has no places to spare.
    bfloat16 with `seq_len` (int32 [n_seq]) runs on the tensor cores; float32 runs the CUDA-core kernel, which is
    exact 32-bit."""
    T = qkv.shape[0]
    if qkv.dtype == torch.bfloat16 and seq_len is not None and tensor_cores:
        return _attn_prefill_mma(qkv, seq_first_row, seq_len, out, nq, nkv, hd, scale, cap, window, kv_src,
                                 kv_row_heads, kv_k_head0, scratch,
                                 (seq_start, seq_slot, kpool, vpool, page_table, ring_len), host_lens)
    if kv_src is None:
        _t(qkv, "qkv", _FLOATS, (T, nq + 2 * nkv, hd))
        kv_src, kv_row_heads, kv_k_head0 = qkv, nq + 2 * nkv, nq
    else:
        _t(qkv, "qkv", _FLOATS, (T, None, hd))
        if qkv.shape[1] < nq:
            raise KernelError("attn_prefill: query rows hold fewer heads than nq")
    q_row_heads = qkv.shape[1]
    _t(kv_src, "kv_src", qkv.dtype, (T, kv_row_heads, hd))
    if kv_k_head0 + 2 * nkv > kv_row_heads:
        raise KernelError("attn_prefill: key/value heads lie outside the rows of kv_src")
    _t(out, "out", qkv.dtype, (T, nq * hd))
    cached = _cached_args("attn_prefill", seq_start, seq_slot, kpool, vpool, page_table, ring_len, qkv.dtype,
                          seq_first_row.numel(), nkv, hd)
    lib = attention_lib(hd)
    _check(lib, lib.janis_attn_prefill(qkv.data_ptr(), kv_src.data_ptr(), _DT[qkv.dtype],
                                       _t(tok_pos, "tok_pos", torch.int32), _t(tok_seq, "tok_seq", torch.int32),
                                       _t(seq_first_row, "seq_first_row", torch.int32), out.data_ptr(), T, nq, nkv,
                                       q_row_heads, kv_row_heads, kv_k_head0, float(scale), float(cap),
                                       int(window), *cached, _stream()))
    return out


def _attn_prefill_mma(qkv, seq_first_row, seq_len, out, nq, nkv, hd, scale, cap, window, kv_src, kv_row_heads,
                      kv_k_head0, scratch=None, cached=(None,) * 5 + (0,), host_lens=None):
    T = qkv.shape[0]
    if kv_src is None:
        _t(qkv, "qkv", torch.bfloat16, (T, nq + 2 * nkv, hd))
        kv_src, kv_row_heads, kv_k_head0 = qkv, nq + 2 * nkv, nq
    else:
        _t(qkv, "qkv", torch.bfloat16, (T, None, hd))
        if qkv.shape[1] < nq:
            raise KernelError("attn_prefill: query rows hold fewer heads than nq")
    _t(kv_src, "kv_src", torch.bfloat16, (T, kv_row_heads, hd))
    if kv_k_head0 + 2 * nkv > kv_row_heads:
        raise KernelError("attn_prefill: key/value heads lie outside the rows of kv_src")
    _t(out, "out", torch.bfloat16, (T, nq * hd))
    n_seq = seq_len.numel()
    _t(seq_len, "seq_len", torch.int32, (n_seq,))
    _t(seq_first_row, "seq_first_row", torch.int32, (n_seq,))
    cached = _cached_args("attn_prefill", *cached, torch.bfloat16, n_seq, nkv, hd)
    lib = attention_lib(hd)
    bm = lib.janis_attn_prefill_tile()      # queries per CTA
    if host_lens is not None:               # the tokens each sequence brings, when the host knows them: no places to spare
        if len(host_lens) != n_seq or sum(host_lens) > T:
            raise KernelError(f"attn_prefill: host_lens {list(host_lens)} do not fit {n_seq} sequences of {T} tokens")
        tiles = sum((int(n) + bm - 1) // bm for n in host_lens)
    else:
        tiles = (T + bm - 1) // bm + n_seq  # >= sum of ceil(len / bm)
    need = int(lib.janis_attn_prefill_scratch(tiles, nq))
    if scratch is not None and (need == 0 or scratch.numel() < need):
        scratch = None
    _check(lib, lib.janis_attn_prefill_mma(qkv.data_ptr(), kv_src.data_ptr(), T, seq_first_row.data_ptr(),
                                           seq_len.data_ptr(), n_seq, tiles, out.data_ptr(), nq, nkv,
                                           qkv.shape[1], kv_row_heads, kv_k_head0, float(scale), float(cap),
                                           int(window), _t(scratch, "scratch", torch.float32) if scratch is not None else None,
                                           scratch.numel() if scratch is not None else 0, *cached,
                                           max(int(n) for n in host_lens) if host_lens else 0, _stream()))
    global _launches
    _launches += int(lib.janis_attn_prefill_kernels()) - 1     # the merge, when tiles were shared
    return out


def attn_set_prefill_kernel(hd: int, which: int = 1) -> None:
    """Choose the bfloat16 prompt kernel of the head size's library: 1 = tcgen05 with the accumulators in
    tensor memory where the head size allows it (a multiple of 64 up to 256; the default), in the form that suits
    the step's size; 2 = always a CTA per tile of queries and head; 3 = always CTAs that stay and take one tile of
    queries after another; 0 = mma.sync."""
    lib = attention_lib(hd)
    lib.janis_attn_set_prefill_kernel(1 if which else 0)
    lib.janis_attn_set_prefill_items({2: 0, 3: 2}.get(which, 1))


def attn_set_prefill_piece(hd: int, piece: int = 0) -> None:
    """Fix how many key tiles a piece of a shared tile of queries holds in the bfloat16 prompt kernels of the
    head size's library (0: chosen from the step's size, the default).  For tests and tuning."""
    attention_lib(hd).janis_attn_set_prefill_piece(int(piece))


def attn_prefill_piece(hd: int, n_tok: int, n_seq: int, nq: int, window: int = 0, tc05: bool = True) -> int:
    """The piece (in key tiles) that a prompt step of these sizes would cut its shared tiles of queries into."""
    lib = attention_lib(hd)
    bm = int(lib.janis_attn_prefill_tile())
    return int(lib.janis_attn_prefill_piece(n_tok, n_seq, (n_tok + bm - 1) // bm + n_seq, nq, window, 1 if tc05 else 0))


def attn_tc05_timeouts(hd: int) -> int:
    """How often a CTA of the tcgen05 prompt kernel has given up a wait (0 unless something is badly wrong)."""
    return int(attention_lib(hd).janis_attn_tc05_timeouts())


def attn_set_decode_wide(hd: int, on: bool = True) -> None:
    """Whether the tensor-core decode kernel of a head size above 128 takes stages of 64 keys in launches of no more
    CTAs than SMs (the default) or stages of 32 keys always.  For tests and tuning."""
    attention_lib(hd).janis_attn_set_decode_wide(1 if on else 0)


def attn_set_decode_kernel(hd: int, which: int = 2) -> None:
    """Choose the decode kernel of the head size's library: 2 = staged by bulk copies with the scores on the
    tensor cores (bfloat16 and head sizes <= 256; the default), 1 = staged, CUDA cores (also what float32
    runs), 0 = straight from global memory into registers."""
    attention_lib(hd).janis_attn_set_decode_kernel(int(which))
    _decode_kernel[hd] = int(which)


def attn_decode_resident(hd: int, dtype, n_ctas: int, sm_count: int) -> int:
    """CTAs of a decode-attention launch of n_ctas CTAs that the GPU holds at once: the bfloat16 tensor-core kernel
    runs with two stages and three CTAs an SM when a launch has more CTAs than two an SM would hold, else with three
    stages and two CTAs an SM; the other kernels hold two."""
    if dtype == torch.bfloat16 and hd <= 256 and _decode_kernel.get(hd, 2) == 2:
        return (3 if attention_lib(hd).janis_attn_decode_stages(int(n_ctas)) == 2 else 2) * sm_count
    return 2 * sm_count


def attn_set_decode_stages(hd: int, stages: int = 0) -> None:
    """Fix the stages of the bfloat16 tensor-core decode kernel (2 or 3; 0: chosen per launch, the default).  For tests."""
    attention_lib(hd).janis_attn_set_decode_stages(int(stages))


def attn_wait_timeouts(hd: int) -> int:
    """How often a decode CTA gave up waiting for its bulk copies (0 in a healthy run); synchronises."""
    return int(attention_lib(hd).janis_attn_wait_timeouts())


def attn_wait_probe(hd: int, tries: int = 64) -> int:
    """Runs the kernels' bounded wait on a barrier that nothing completes: returns 1 when the wait gave up
    (as it must) and the kernel returned.  Raises the library's counter of timeouts by one."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = attention_lib(hd)
    _check(lib, lib.janis_attn_wait_probe(int(tries), status.data_ptr(), _stream()))
    return int(status.item())


def attn_decode_scratch_floats(n_seq: int, nq: int, hd: int, max_chunks: int) -> int:
    return n_seq * nq * max_chunks * (hd + 2)


_decode_kernel: dict[int, int] = {}      # head size -> kernel chosen for tests (default 2)


def attn_decode(qkv, kpool, vpool, page_table, seq_slot, seq_len, scratch, out, nq: int, nkv: int, hd: int,
                scale: float, cap: float, window: int, ring_len: int, chunk: int, max_chunks: int):
    """One query per sequence over the paged cache.  qkv: [n_seq, heads >= nq, hd] with q first;
    seq_len counts the new token; scratch is float32.  The chunks of a sequence are merged by a second
    kernel; a launch of one chunk per sequence (max_chunks == 1) on the bfloat16 tensor-core kernel
    writes the result itself."""
    n_seq = qkv.shape[0]
    _t(qkv, "qkv", _FLOATS, (n_seq, None, hd))
    if qkv.shape[1] < nq:
        raise KernelError("attn_decode: query rows hold fewer heads than nq")
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(vpool, "vpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(page_table, "page_table", torch.int32, (None, None))
    _t(scratch, "scratch", torch.float32)
    _t(out, "out", qkv.dtype, (n_seq, nq * hd))
    if seq_slot.numel() < n_seq or seq_len.numel() < n_seq:
        raise KernelError("attn_decode: sequence tables shorter than the batch")
    lib = attention_lib(hd)
    direct = max_chunks == 1 and qkv.dtype == torch.bfloat16 and hd <= 256 and _decode_kernel.get(hd, 2) == 2
    _check(lib, lib.janis_attn_decode(qkv.data_ptr(), kpool.data_ptr(), vpool.data_ptr(), _DT[qkv.dtype],
                                      page_table.data_ptr(), page_table.shape[1],
                                      _t(seq_slot, "seq_slot", torch.int32), _t(seq_len, "seq_len", torch.int32),
                                      scratch.data_ptr(), scratch.numel(), out.data_ptr(), n_seq, nq, nkv,
                                      qkv.shape[1], float(scale), float(cap), int(window), int(ring_len),
                                      int(chunk), int(max_chunks), _stream()), kernels=1 if direct else 2)
    return out


# ---------------------------------------------------------------------------
# mixers with run-time sizes: attention with mixed heads, gated linear attention
# ---------------------------------------------------------------------------

def qkv_rotate_store(rows, tok_pos, tok_seq, seq_slot, inv_qk, rot: int, inv_v, H: int, G: int, d: int, dv: int,
                     kpool=None, vpool=None, page_table=None, store: bool = True):
    """Rotary encoding of the first `rot` features of the queries and keys of a step (pairs i, i + rot/2), rotation
    of the values over all dv features by inv_v (None: values stay as projected), and the write of keys and values
    into the paged cache line.  rows [T, H d + G d + G dv] holds q, then k, then v; with store=False the rows hold q
    alone.  kpool [pages, G, PAGE, d], vpool [pages, G, PAGE, dv]."""
    T, width = rows.shape
    _t(rows, "rows", _FLOATS, (T, None))
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("qkv_rotate_store: position tables shorter than the step")
    _t(inv_qk, "inv_qk", torch.float32, (rot // 2,))
    if inv_v is not None:
        _t(inv_v, "inv_v", torch.float32, (dv // 2,))
    stride = 0
    if store:
        n_pages = kpool.shape[0]
        _t(kpool, "kpool", rows.dtype, (n_pages, G, PAGE, d))
        _t(vpool, "vpool", rows.dtype, (n_pages, G, PAGE, dv))
        _t(page_table, "page_table", torch.int32, (None, None))
        _t(seq_slot, "seq_slot", torch.int32)
        stride = page_table.shape[1]
    lib = mixers()
    _check(lib, lib.janis_qkv_rotate_store(
        rows.data_ptr(), _DT[rows.dtype], width, _t(tok_pos, "tok_pos", torch.int32), _t(tok_seq, "tok_seq", torch.int32),
        seq_slot.data_ptr() if store else None, inv_qk.data_ptr() if rot else None, rot,
        inv_v.data_ptr() if inv_v is not None else None, T, H, G, d, dv, 1 if store else 0,
        kpool.data_ptr() if store else None, vpool.data_ptr() if store else None,
        page_table.data_ptr() if store else None, stride, _stream()))
    return rows


def talk_attention(q_rows, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, talk, inv_v, out, H: int, G: int,
                   d: int, dv: int, scale: float, block: int = 0, sink: bool = False, one_row: bool = False,
                   max_keys: int = 0, n_chunks: int = 1, scratch=None, window: int = 0, cap: float = 0.0,
                   sink_values=None, mix_after: bool = False, values_in_keys: bool = False, stats=None, keep_first: int = 0):
    """Causal attention of every token of the step over its sequence's cache line (which already holds the step's
    own keys and values).  The scaled scores of the H query heads are mixed by talk [H, H] float32 (None: left
    alone) before the softmax; with block > 0 a key is seen only inside the query's block of that many positions;
    with window > 0 only among the query's last `window` positions (its own included); with sink, 1 is added to the softmax's denominator; with inv_v each head's output is turned back by the query's
    position (the cached values were rotated by theirs).  q_rows [T, >= H d], out [T, H dv].
    bfloat16 with d a multiple of 16, dv a multiple of 8 and up to 32 heads runs on the tensor cores (a CTA per 16
    or 8 rows of the step; one_row=True, for decode steps, gives every row a CTA of its own); everything else
    runs the plain kernel, which is exact 32-bit for float32.  A decode step on the tensor cores may cut every row's
    keys over n_chunks CTAs (max_keys: a bound on the keys a row sees; scratch: float32, at least
    `talk_attention_scratch_floats`) whose shares a second kernel puts together.
    cap > 0: every scaled score becomes cap tanh(score / cap) first.  sink_values [H] float32 (with sink): exp of
    head h's value joins its denominator instead of 1.  mix_after: talk mixes the heads' weights after the softmax
    instead of their scores before it, which takes two passes over the keys and `stats`, float32 of at least
    `talk_attention_stats_floats` (the rows' maxima and denominators between the passes).  values_in_keys: the
    values are the first dv features of the cached keys (vpool is not read and may be None).  keep_first (with a
    window): the sequence's first `keep_first` positions stay seen behind the window, at their true positions; a bound
    `max_keys` then counts them too."""
    T = q_rows.shape[0]
    _t(q_rows, "q_rows", _FLOATS, (T, None))
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", q_rows.dtype, (n_pages, G, PAGE, d))
    if not values_in_keys:
        _t(vpool, "vpool", q_rows.dtype, (n_pages, G, PAGE, dv))
    if sink_values is not None and not sink:
        raise KernelError("talk_attention: sink values without a sink")
    two_pass = bool(mix_after) and talk is not None
    _t(page_table, "page_table", torch.int32, (None, None))
    _t(out, "out", q_rows.dtype, (T, H * dv))
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("talk_attention: position tables shorter than the step")
    lib = mixers()
    _check(lib, lib.janis_talk_attention(
        q_rows.data_ptr(), _DT[q_rows.dtype], q_rows.shape[1], _t(tok_pos, "tok_pos", torch.int32),
        _t(tok_seq, "tok_seq", torch.int32), _t(seq_slot, "seq_slot", torch.int32), kpool.data_ptr(),
        None if values_in_keys else vpool.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        _t(talk, "talk", torch.float32, (H, H)) if talk is not None else None,
        _t(inv_v, "inv_v", torch.float32, (dv // 2,)) if inv_v is not None else None, out.data_ptr(), T, H, G, d, dv,
        float(scale), int(block), 1 if sink else 0, 1 if one_row else 0, int(max_keys), int(n_chunks),
        _t(scratch, "scratch", torch.float32) if scratch is not None else None,
        scratch.numel() if scratch is not None else 0, int(window), float(cap),
        _t(sink_values, "sink_values", torch.float32, (H,)) if sink_values is not None else None,
        1 if mix_after else 0, 1 if values_in_keys else 0,
        _t(stats, "stats", torch.float32) if stats is not None else None, stats.numel() if stats is not None else 0,
        int(keep_first), _stream()),
        kernels=(2 if two_pass else 1) *
                (2 if (one_row and n_chunks > 1 and scratch is not None and q_rows.dtype == torch.bfloat16) else 1))
    return out


def talk_attention_rows_floats(dtype, T: int, H: int, G: int, d: int, dv: int, max_keys: int) -> int:
    """Floats of scratch that `talk_attention_rows` wants for a step of T rows that see up to max_keys keys each, or 0
    where it does not take the sizes (heads that are no multiples of 16 bytes; scores of a chunk beyond shared memory)."""
    return int(mixers().janis_talk_attention_rows_floats(_DT[dtype], int(T), int(H), int(G), int(d), int(dv), int(max_keys)))


def talk_attention_rows(q_rows, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, talk, out, H: int, G: int, d: int,
                        dv: int, scale: float, scratch, max_keys: int, sink: bool = False, window: int = 0, cap: float = 0.0,
                        sink_values=None, values_in_keys: bool = False, keep_first: int = 0):
    """`talk_attention` for a decode step (every row a query position of a sequence of its own): keys and values are
    read once, 16 bytes a lane, a CTA per row and chunk of keys; scores are capped (cap > 0), seen inside the window
    (window > 0), softmaxed with the sink (sink; sink_values [H] float32: learnt ones) and, with talk [H, H] float32,
    the heads' weights mixed after the softmax; values_in_keys: the values are the first dv features of the keys.
    q_rows [T, >= H d], out [T, H dv]; max_keys bounds the keys a row sees; scratch float32 of at least
    `talk_attention_rows_floats`.  keep_first (with a window): the sequence's first positions that stay seen behind the
    window; max_keys counts them too.  Sums are float and their order depends on the row alone."""
    T = q_rows.shape[0]
    _t(q_rows, "q_rows", _FLOATS, (T, None))
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", q_rows.dtype, (n_pages, G, PAGE, d))
    if not values_in_keys:
        _t(vpool, "vpool", q_rows.dtype, (n_pages, G, PAGE, dv))
    if sink_values is not None and not sink:
        raise KernelError("talk_attention_rows: sink values without a sink")
    _t(page_table, "page_table", torch.int32, (None, None))
    _t(out, "out", q_rows.dtype, (T, H * dv))
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("talk_attention_rows: position tables shorter than the step")
    lib = mixers()
    _check(lib, lib.janis_talk_attention_rows(
        q_rows.data_ptr(), _DT[q_rows.dtype], q_rows.shape[1], _t(tok_pos, "tok_pos", torch.int32),
        _t(tok_seq, "tok_seq", torch.int32), _t(seq_slot, "seq_slot", torch.int32), kpool.data_ptr(),
        None if values_in_keys else vpool.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        _t(talk, "talk", torch.float32, (H, H)) if talk is not None else None, out.data_ptr(), T, H, G, d, dv,
        float(scale), 1 if sink else 0, int(max_keys), int(window), float(cap),
        _t(sink_values, "sink_values", torch.float32, (H,)) if sink_values is not None else None,
        1 if values_in_keys else 0, _t(scratch, "scratch", torch.float32), scratch.numel(), int(keep_first), _stream()), kernels=4)
    return out


def talk_attention_stats_floats(T: int, H: int) -> int:
    """What `talk_attention(mix_after=True)` keeps between its passes: a maximum and a denominator per row and head."""
    return 2 * T * H


def talk_attention_scratch_floats(T: int, n_chunks: int, H: int, dv: int) -> int:
    return T * n_chunks * H * (dv + 2) if n_chunks > 1 else 0


def talk_attention_set_kernel(which: int = 1) -> None:
    """1: the tensor-core kernel where the sizes allow it (the default); 0: the plain kernel always.  For tests."""
    mixers().janis_talk_attention_set_kernel(int(which))


def gla_scan(rows, q_off: int, k_off: int, v_off: int, z, z_bias, seq_slot, seq_first_row, seq_start, seq_end, state,
             o_out, n_seq: int, H: int, d: int, dv: int, q_scale: float, tau: float, decay=None):
    """The recurrence of gated linear attention over the tokens each sequence brings to the step, in order:
    a = sigmoid(z + z_bias)^(1/tau) per key channel, S = diag(a) S + k v^T, o = S^T (q q_scale).
    rows [T, width] holds the projections (q [H, d] at q_off, k at k_off, v [H, dv] at v_off), z [T, H d] the
    projected decay logits; state float32 [slots, H, dv, d] (a column's key channels side by side) is read and written back for sequences whose slot is
    >= 0; o_out float32 [T, H dv]; decay float32 [T, H d] receives the decays (a kernel of its own forms them once
    for all the CTAs of a head; allocated here when not given)."""
    T, width = rows.shape
    if decay is None:
        decay = torch.empty((T, H * d), dtype=torch.float32, device=rows.device)
    _t(decay, "decay", torch.float32, (T, H * d))
    _t(rows, "rows", _FLOATS, (T, None))
    _t(z, "z", rows.dtype, (T, H * d))
    _t(z_bias, "z_bias", rows.dtype, (H * d,))
    _t(state, "state", torch.float32, (None, H, dv, d))
    _t(o_out, "o_out", torch.float32, (T, H * dv))
    for name, tab in (("seq_slot", seq_slot), ("seq_first_row", seq_first_row), ("seq_start", seq_start), ("seq_end", seq_end)):
        _t(tab, name, torch.int32)
        if tab.numel() < n_seq:
            raise KernelError(f"gla_scan: {name} shorter than the step's sequences")
    lib = mixers()
    _check(lib, lib.janis_gla_scan(rows.data_ptr(), _DT[rows.dtype], width, q_off, k_off, v_off, z.data_ptr(),
                                   z_bias.data_ptr(), decay.data_ptr(), T, seq_slot.data_ptr(), seq_first_row.data_ptr(),
                                   seq_start.data_ptr(), seq_end.data_ptr(), state.data_ptr(), o_out.data_ptr(), n_seq,
                                   H, d, dv, float(q_scale), float(tau), _stream()), kernels=2)
    return o_out


def head_norm_gate(o, rows, g_off: int, weight, eps: float, out, H: int, dv: int, gate: str = "silu"):
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * silu(gate[t, h]) per head of dv features; the gate
    is read from rows [T, width] at g_off (rows None: no gate; gate="sigmoid": the logistic function alone).  o float32
    [T, H dv]; weight float32 [dv], one vector for all heads, or [H dv] with a run per head."""
    T = o.shape[0]
    if gate not in ("silu", "sigmoid"):
        raise KernelError(f"head_norm_gate: unknown gate {gate!r}")
    _t(o, "o", torch.float32, (T, H * dv))
    per_head = weight.numel() == H * dv and H > 1
    _t(weight, "weight", torch.float32, (H * dv,) if per_head else (dv,))
    _t(out, "out", _FLOATS, (T, H * dv))
    if rows is not None:
        _t(rows, "rows", out.dtype, (T, None))
    lib = mixers()
    _check(lib, lib.janis_head_norm_gate(o.data_ptr(), rows.data_ptr() if rows is not None else None, _DT[out.dtype],
                                         rows.shape[1] if rows is not None else 0, g_off, weight.data_ptr(), float(eps),
                                         out.data_ptr(), T, H, dv, 1 if per_head else 0, 1 if gate == "sigmoid" else 0,
                                         _stream()))
    return out


def mlstm_scan(rows, q_off: int, k_off: int, v_off: int, z, bias, cap: float, seq_slot, seq_first_row, seq_start, seq_end,
               state_c, state_n, state_m, o_out, n_seq: int, H: int, d: int, dv: int, q_scale: float, coef):
    """The matrix memory with exponential gates over a step's tokens, sequence by sequence in order.  rows [T, width]
    holds q [H, d], k [H, d] and v [H, dv] at their offsets; z float32 [T, 2 H] the input gates' logits, then the forget
    gates'; bias float32 [2 H]; with i = cap tanh((zi + bi) / cap), f = logsigmoid(cap tanh((zf + bf) / cap)):
    m' = max(f + m, i); C <- e^(f + m - m') C + e^(i - m') k v^T; n likewise with k alone;
    o = C^T (q q_scale) / (max(|n . q q_scale|, e^(-m')) + 1e-6).  The cache parts (float32): state_c [slots, H, dv, d]
    (C transposed), state_n [slots, H, ceil(dv / 8), d] (a copy of n per group of 8 value columns), state_m [slots, H].
    coef: float32 scratch [T, H, 3]; o_out float32 [T, H dv].  Sequences without a slot start from zero and store nothing."""
    T = rows.shape[0]
    _t(rows, "rows", _FLOATS, (T, None))
    _t(z, "z", torch.float32, (T, 2 * H))
    _t(bias, "bias", torch.float32, (2 * H,))
    _t(coef, "coef", torch.float32, (T, H, 3))
    _t(o_out, "o_out", torch.float32, (T, H * dv))
    n_slots = state_c.shape[0]
    _t(state_c, "state_c", torch.float32, (n_slots, H, dv, d))
    _t(state_n, "state_n", torch.float32, (n_slots, H, (dv + 7) // 8, d))
    _t(state_m, "state_m", torch.float32, (n_slots, H))
    if max(q_off + H * d, k_off + H * d, v_off + H * dv) > rows.shape[1]:
        raise KernelError("mlstm_scan: the projections do not fit the rows")
    lib = mixers()
    _check(lib, lib.janis_mlstm_scan(rows.data_ptr(), _DT[rows.dtype], rows.shape[1], q_off, k_off, v_off, z.data_ptr(),
                                     bias.data_ptr(), float(cap), coef.data_ptr(), T, _t(seq_slot, "seq_slot", torch.int32),
                                     _t(seq_first_row, "seq_first_row", torch.int32), _t(seq_start, "seq_start", torch.int32),
                                     _t(seq_end, "seq_end", torch.int32), state_c.data_ptr(), state_n.data_ptr(),
                                     state_m.data_ptr(), o_out.data_ptr(), n_seq, H, d, dv, float(q_scale), _stream()),
           kernels=2)
    return o_out


def hc_spread(x, h, copies: int):
    """h[t, s] = x[t] for every copy s of the stream; x float32 [T, W], h float32 [T, copies W]."""
    T, W = x.shape
    lib = mixers()
    _check(lib, lib.janis_hc_spread(_t(x, "x", torch.float32, (T, W)), _t(h, "h", torch.float32, (T, copies * W)), T,
                                    int(copies), W, _stream()))
    return h


def hc_read_norm(h, copies: int, a, weight, eps: float, out, rows=None):
    """out[r] = norm(sum_s a[s] h[row, s]) with norm(u) = u / sqrt(mean(u^2) + eps) * weight; h float32 [T, copies W],
    a float32 [copies] (None: ones, the plain sum of the copies), weight float32 [W] (offset + w), rows: the rows to
    read (None: all)."""
    R, W = out.shape
    if rows is None and h.shape[0] != R:
        raise KernelError(f"hc_read_norm: {h.shape[0]} input rows for {R} output rows")
    lib = mixers()
    _check(lib, lib.janis_hc_read_norm(_t(h, "h", torch.float32, (None, copies * W)),
                                       _t(rows, "rows", torch.int32, (R,)) if rows is not None else None,
                                       _t(a, "a", torch.float32, (copies,)) if a is not None else None,
                                       _t(weight, "weight", torch.float32, (W,)), float(eps), _t(out, "out", _FLOATS, (R, W)),
                                       _DT[out.dtype], R, int(copies), W, _stream()))
    return out


def hc_update(h, res, copies: int, mix, b, a_next=None, w_next=None, eps_next: float = 0.0, out=None):
    """h[t, k] <- sum_s mix[s, k] h[t, s] + b[k] res[t] for all copies k at once (float32, in place); with a_next and
    w_next also out[t] = norm(sum_k a_next[k] h[t, k]; w_next), the next sublayer's read, in the same pass.
    h float32 [T, copies W], res [T, W] in the activation type, mix float32 [copies, copies] ([from, to]), b [copies]."""
    T, W = res.shape
    fused = w_next is not None
    lib = mixers()
    _check(lib, lib.janis_hc_update(_t(h, "h", torch.float32, (T, copies * W)), _t(res, "res", _FLOATS, (T, W)), _DT[res.dtype],
                                    _t(mix, "mix", torch.float32, (copies, copies)), _t(b, "b", torch.float32, (copies,)),
                                    _t(a_next, "a_next", torch.float32, (copies,)) if fused else None,
                                    _t(w_next, "w_next", torch.float32, (W,)) if fused else None, float(eps_next),
                                    _t(out, "out", res.dtype, (T, W)) if fused else None, T, int(copies), W, _stream()))
    return out if fused else None


# ---------------------------------------------------------------------------
# Dynamic Tanh, state-space mixers, branches side by side, mixture of experts
# ---------------------------------------------------------------------------

def dyt_norm(h, res, alpha: float, weight, bias, out, rows=None):
    """h += res (when res is given: the float32 residual sum, in place), then out[r] = tanh(alpha h[rows[r] or r]) *
    weight + bias.  h float32 [T, H]; res [T, H] float32 or bfloat16 (not together with rows); weight, bias float32."""
    H = h.shape[-1]
    R = out.shape[0]
    if rows is None and h.shape[0] != R:
        raise KernelError(f"dyt_norm: {h.shape[0]} input rows for {R} output rows")
    lib = mixers()
    _check(lib, lib.janis_dyt_norm(_t(h, "h", torch.float32, (None, H)),
                                   _t(res, "res", _FLOATS, (R, H)) if res is not None else None,
                                   _DT[res.dtype] if res is not None else 0,
                                   _t(rows, "rows", torch.int32, (R,)) if rows is not None else None, float(alpha),
                                   _t(weight, "weight", torch.float32, (H,)), _t(bias, "bias", torch.float32, (H,)),
                                   _t(out, "out", _FLOATS, (R, H)), _DT[out.dtype], R, H, _stream()))
    return out


def causal_conv_silu(rows, col_off: int, channels: int, weight, bias, state, tok_seq, seq_slot, seq_first_row, seq_start,
                     seq_end, n_seq: int, out, one_token: bool = False, act: bool = True):
    """out[t, c] = silu(bias[c] + sum_j weight[c, K-1-j] x[t-j, c]) (act=False: without the silu; bias None: without
    one) over the channels rows[:, col_off : col_off +
    channels] of each sequence's tokens; inputs before the step come from state float32 [slots, max(K-1, 1), channels]
    (the last K-1 inputs of each slot), which is brought up to date: by the same kernel for sequences that bring one
    token, by a second kernel for the others (one_token=True: every sequence brings one, a decode step, and the
    second kernel is not launched).  Sequences without a slot start from zeros and store nothing.  weight float32
    [channels, K], bias float32 [channels]."""
    T, width = rows.shape
    K = weight.shape[1]
    _t(rows, "rows", _FLOATS, (T, None))
    _t(state, "state", torch.float32, (None, max(K - 1, 1), channels))
    for name, tab, n in (("tok_seq", tok_seq, T), ("seq_slot", seq_slot, n_seq), ("seq_first_row", seq_first_row, n_seq),
                         ("seq_start", seq_start, n_seq), ("seq_end", seq_end, n_seq)):
        _t(tab, name, torch.int32)
        if tab.numel() < n:
            raise KernelError(f"causal_conv_silu: {name} shorter than the step")
    lib = mixers()
    _check(lib, lib.janis_causal_conv_silu(rows.data_ptr(), _DT[rows.dtype], width, int(col_off), int(channels), K,
                                           _t(weight, "weight", torch.float32, (channels, K)),
                                           _t(bias, "bias", torch.float32, (channels,)) if bias is not None else None,
                                           state.data_ptr(),
                                           tok_seq.data_ptr(), seq_slot.data_ptr(), seq_first_row.data_ptr(),
                                           seq_start.data_ptr(), seq_end.data_ptr(), T, n_seq, 1 if one_token else 0,
                                           _t(out, "out", rows.dtype, (T, channels)), 1 if act else 0, _stream()),
           kernels=2 if K > 1 and not one_token else 1)
    return out


def selective_scan(u, u_off: int, dt, dt_off: int, dt_bias, A, a_per_state: bool, bc, b_off: int, c_off: int, D, z,
                   z_off: int, seq_slot, seq_first_row, seq_start, seq_end, n_seq: int, state, out, C: int, N: int,
                   ch_per_head: int, ch_per_group: int, scratch=None):
    """The recurrence S[c, n] <- exp(delta A) S[c, n] + delta u[c] B[n], o[c] = sum_n S[c, n] C[n] + D u[c] over the
    tokens each sequence brings, in order, with delta = softplus(dt + dt_bias).  u [T, *] holds the channels at
    u_off; dt [T, *] one step size per head (c // ch_per_head) at dt_off; bc [T, *] holds B at b_off and C at c_off,
    N numbers per group (c // ch_per_group); A float32 is [heads, N] (a_per_state) or [heads]; dt_bias, D float32
    [heads].  With z ([T, *], the gate's channels at z_off) out [T, C] takes o * silu(z) in the activations' type;
    without, out is float32 o.  state float32 [slots, C, N] is read and written back for slots >= 0.  A first kernel
    forms delta (and, with one A per head, exp(delta A) - 1) once per (token, head) into scratch (float32, at least
    `selective_scan_scratch_floats`; allocated here when not given)."""
    T = u.shape[0]
    heads = C // ch_per_head
    dtype = u.dtype
    for name, x in (("u", u), ("dt", dt), ("bc", bc)) + ((("z", z),) if z is not None else ()):
        _t(x, name, dtype, (T, None))
    _t(dt_bias, "dt_bias", torch.float32, (heads,))
    _t(A, "A", torch.float32, (heads, N) if a_per_state else (heads,))
    _t(D, "D", torch.float32, (heads,))
    _t(state, "state", torch.float32, (None, C, N))
    _t(out, "out", dtype if z is not None else torch.float32, (T, C))
    if u_off + C > u.shape[1] or dt_off + heads > dt.shape[1] or max(b_off, c_off) + (C // ch_per_group) * N > bc.shape[1] \
            or (z is not None and z_off + C > z.shape[1]):
        raise KernelError("selective_scan: a column range lies outside its rows")
    for name, tab in (("seq_slot", seq_slot), ("seq_first_row", seq_first_row), ("seq_start", seq_start), ("seq_end", seq_end)):
        _t(tab, name, torch.int32)
        if tab.numel() < n_seq:
            raise KernelError(f"selective_scan: {name} shorter than the step's sequences")
    need = selective_scan_scratch_floats(T, heads)
    if scratch is None:
        scratch = torch.empty((need,), dtype=torch.float32, device=u.device)
    _t(scratch, "scratch", torch.float32)
    if scratch.numel() < need:
        raise KernelError(f"selective_scan: scratch of {scratch.numel()} floats, {need} wanted")
    lib = mixers()
    _check(lib, lib.janis_selective_scan(
        u.data_ptr(), _DT[dtype], u.shape[1], int(u_off), dt.data_ptr(), dt.shape[1], int(dt_off), dt_bias.data_ptr(),
        A.data_ptr(), 1 if a_per_state else 0, bc.data_ptr(), bc.shape[1], int(b_off), int(c_off), D.data_ptr(),
        z.data_ptr() if z is not None else None, z.shape[1] if z is not None else 0, int(z_off), seq_slot.data_ptr(),
        seq_first_row.data_ptr(), seq_start.data_ptr(), seq_end.data_ptr(), n_seq, state.data_ptr(), out.data_ptr(),
        C, N, int(ch_per_head), int(ch_per_group), T, scratch.data_ptr(), _stream()), kernels=2)
    return out


def selective_scan_scratch_floats(n_tok: int, heads: int) -> int:
    return 2 * n_tok * heads


def selective_scan_set_lanes(lanes: int = 0) -> None:
    """Fix how many lanes share a channel in `selective_scan` (4, 8, 16 or 32; 0: chosen per launch, the default).
    For tests and tuning."""
    mixers().janis_selective_scan_set_lanes(int(lanes))


def selective_scan_set_form(form: int = 0) -> None:
    """0: a step in which a sequence brings several tokens runs the form that stages tiles of B and C in shared memory
    where the sizes allow it and there are 64 states a channel or more (the default); 1: always the form that keeps a
    tile's inputs in registers; 2: the staged form wherever the sizes allow it.  For tests."""
    mixers().janis_selective_scan_set_form(int(form))


def gate_group_norm(o, rows, z_off: int, weight, eps: float, n_groups: int, out):
    """out = rms(o * silu(z)) * weight, the root mean square taken over each of n_groups equal parts of a row;
    o float32 [T, C], z = rows[:, z_off : z_off + C], weight float32 [C]."""
    T, C = o.shape
    _t(o, "o", torch.float32, (T, C))
    _t(rows, "rows", out.dtype, (T, None))
    if z_off + C > rows.shape[1]:
        raise KernelError("gate_group_norm: the gate lies outside its rows")
    lib = mixers()
    _check(lib, lib.janis_gate_group_norm(o.data_ptr(), rows.data_ptr(), _DT[out.dtype], rows.shape[1], int(z_off),
                                          _t(weight, "weight", torch.float32, (C,)), float(eps), int(n_groups),
                                          _t(out, "out", _FLOATS, (T, C)), T, C, _stream()))
    return out


def rmsnorm_accumulate(x, weight, eps: float, scale: float, acc, first: bool = False):
    """acc = (0 if first else acc) + scale * x / sqrt(mean(x^2) + eps) * weight; x [T, H], acc float32 [T, H]."""
    T, H = x.shape
    lib = mixers()
    _check(lib, lib.janis_rmsnorm_accumulate(_t(x, "x", _FLOATS, (T, H)), _DT[x.dtype], _t(weight, "weight", torch.float32, (H,)),
                                             float(eps), float(scale), _t(acc, "acc", torch.float32, (T, H)),
                                             1 if first else 0, T, H, _stream()))
    return acc


def sigmoid_gate(x, rows, g_off: int, per: int = 1):
    """x[t, c] *= sigmoid(rows[t, g_off + c // per]) in place: a gate per element, or per run of `per` elements (a
    head); x [T, n], rows [T, >= g_off + n / per] of x's dtype."""
    T, n = x.shape
    lib = mixers()
    _check(lib, lib.janis_sigmoid_gate(_t(x, "x", _FLOATS, (T, n)), _t(rows, "rows", x.dtype, (T, None)), _DT[x.dtype],
                                       rows.shape[1], int(g_off), T, n, int(per), _stream()))
    return x


def group_norm(h, res, alpha: float, weight, eps: float, groups: int, out, rows=None):
    """RMS norm in `groups` equal runs of the row, each divided by its own sqrt(mean(run^2) + eps), the whole times
    weight.  With res: h <- norm(alpha h + res) on the float32 stream in place, and out (when given) = h rounded.
    Without: out = norm(h[rows]) (all rows when `rows` is None), h untouched."""
    R = out.shape[0] if out is not None else h.shape[0]
    H = h.shape[1]
    lib = mixers()
    _check(lib, lib.janis_group_norm(_t(h, "h", torch.float32, (None, H)),
                                     _t(res, "res", _FLOATS, (R, H)) if res is not None else None,
                                     _DT[res.dtype] if res is not None else 0,
                                     _t(rows, "rows", torch.int32, (R,)) if rows is not None else None, float(alpha),
                                     _t(weight, "weight", torch.float32, (H,)), float(eps), int(groups),
                                     _t(out, "out", _FLOATS, (R, H)) if out is not None else None,
                                     _DT[out.dtype] if out is not None else 0, R, H, _stream()))
    return out


def round_rows(h, out):
    """out = h rounded to bfloat16 (h float32, same shape)."""
    lib = mixers()
    _check(lib, lib.janis_round_rows(_t(h, "h", torch.float32), _t(out, "out", torch.bfloat16, tuple(h.shape)),
                                     h.numel(), _stream()))
    return out


def qkv_conv_norm_store(rows, H: int, G: int, d: int, dv: int, conv_w, conv_state, wq, wk, v_unit: bool, eps: float,
                        tok_pos, tok_seq, seq_slot, seq_first_row, seq_start, seq_end, n_seq: int, q_out, kpool, vpool,
                        page_table, one_token: bool = False):
    """What an attention does to its projections before it caches them.  rows [T, >= H d + G d + G dv] holds q | k | v.
    conv_w float32 [channels, K] (None: no filter): every channel is filtered over time, y[t] = sum_j conv_w[c, K-1-j]
    x[t-j]; inputs before the step come from conv_state float32 [slots, K-1, channels], which is brought up to date
    (as `causal_conv_silu` does it).  wq [H d], wk [G d] float32 (None: no norm): RMS norm over the whole of q, of k.
    v_unit: every value head is divided by its root mean square.  q goes to q_out [T, H d], k and v into the cache
    line at the tokens' positions; sequences without a slot store nothing."""
    T, width = rows.shape
    C = H * d + G * (d + dv)
    K = conv_w.shape[1] if conv_w is not None else 0
    _t(rows, "rows", _FLOATS, (T, None))
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", rows.dtype, (n_pages, G, PAGE, d))
    _t(vpool, "vpool", rows.dtype, (n_pages, G, PAGE, dv))
    _t(page_table, "page_table", torch.int32, (None, None))
    for name, tab, n in (("tok_pos", tok_pos, T), ("tok_seq", tok_seq, T), ("seq_slot", seq_slot, n_seq),
                         ("seq_first_row", seq_first_row, n_seq), ("seq_start", seq_start, n_seq), ("seq_end", seq_end, n_seq)):
        _t(tab, name, torch.int32)
        if tab.numel() < n:
            raise KernelError(f"qkv_conv_norm_store: {name} shorter than the step")
    if K > 1:
        _t(conv_state, "conv_state", torch.float32, (None, K - 1, C))
    lib = mixers()
    _check(lib, lib.janis_qkv_conv_norm_store(
        rows.data_ptr(), _DT[rows.dtype], width, T, H, G, d, dv, K,
        _t(conv_w, "conv_w", torch.float32, (C, K)) if conv_w is not None else None,
        conv_state.data_ptr() if K > 1 else None,
        _t(wq, "wq", torch.float32, (H * d,)) if wq is not None else None,
        _t(wk, "wk", torch.float32, (G * d,)) if wk is not None else None, 1 if v_unit else 0, float(eps),
        tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), seq_first_row.data_ptr(), seq_start.data_ptr(),
        seq_end.data_ptr(), _t(q_out, "q_out", rows.dtype, (T, H * d)), kpool.data_ptr(), vpool.data_ptr(),
        page_table.data_ptr(), page_table.shape[1], _stream()))
    if K > 1 and not one_token:
        _check(lib, lib.janis_conv_state_update(rows.data_ptr(), _DT[rows.dtype], width, 0, C, K, conv_state.data_ptr(),
                                                seq_slot.data_ptr(), seq_first_row.data_ptr(), seq_start.data_ptr(),
                                                seq_end.data_ptr(), n_seq, _stream()))
    return q_out


def latent_rotate_store(rows, lat_off: int, H: int, d: int, dr: int, R: int, wc, eps: float, inv_freq, amp: float,
                        tok_pos, tok_seq, seq_slot, qfull, kpool, page_table, rot: int | None = None, q_rows=None,
                        halves: bool = False):
    """rows [T, ...]: H query heads of d + dr at 0, the compressed row [c (R) | r (dr)] at lat_off.  c is RMS-normed with
    wc, r and every query head's last dr features are turned by the token's position (pairs 2i, 2i + 1 of the first
    `rot` of them, all when None, angle pos * inv_freq[i], sine and cosine times amp).  [norm(c) | turn(r)] becomes the key of the line's single head at the
    token's position (kpool [pages, 1, PAGE, R + dr]); the turned query parts go to qfull[t, h, R:], whose first R
    features per head are left for the absorbed queries.  q_rows [T, >= H (d + dr)]: the query heads come from these rows
    instead (a product of their own; lat_off then counts from 0 in `rows`).  halves: the turned pairs are (p, p + rot/2)."""
    T, width = rows.shape
    _t(rows, "rows", _FLOATS, (T, None))
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", rows.dtype, (n_pages, 1, PAGE, R + dr))
    _t(page_table, "page_table", torch.int32, (None, None))
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("latent_rotate_store: position tables shorter than the step")
    lib = mixers()
    _check(lib, lib.janis_latent_rotate_store(
        rows.data_ptr(), _DT[rows.dtype], width, int(lat_off),
        _t(q_rows, "q_rows", rows.dtype, (T, None)) if q_rows is not None else None,
        q_rows.shape[1] if q_rows is not None else 0, 1 if halves else 0, T, H, d, dr, dr if rot is None else int(rot), R,
        _t(wc, "wc", torch.float32, (R,)), float(eps), _t(inv_freq, "inv_freq", torch.float32, (max(dr // 2, 1),) if dr < 2 else (dr // 2,)), float(amp),
        _t(tok_pos, "tok_pos", torch.int32), _t(tok_seq, "tok_seq", torch.int32), _t(seq_slot, "seq_slot", torch.int32),
        _t(qfull, "qfull", rows.dtype, (T, H * (R + dr))), kpool.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        _stream()))
    return qfull


def qk_rotate_norm_store(rows, tok_pos, tok_seq, seq_slot, inv_freq, rot: int, halves: bool, unit_norm: bool, eps: float,
                         H: int, G: int, d: int, kpool, vpool, page_table):
    """rows [T, >= (H + G) d]: q (H heads of d), then k (G heads).  The first `rot` features of every head turn by the
    token's position (pairs (2p, 2p + 1), or (p, p + rot/2) with halves; angle pos * inv_freq[p]); with unit_norm every
    head is then divided by sqrt(mean(head^2) + eps).  q is written back in place, k to the line's keys at the token's
    position (kpool [pages, G, PAGE, d]), and k as projected to its values (vpool, the same shape; None: no values)."""
    T = rows.shape[0]
    _t(rows, "rows", _FLOATS, (T, None))
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", rows.dtype, (n_pages, G, PAGE, d))
    if vpool is not None:
        _t(vpool, "vpool", rows.dtype, (n_pages, G, PAGE, d))
    _t(page_table, "page_table", torch.int32, (None, None))
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("qk_rotate_norm_store: position tables shorter than the step")
    lib = mixers()
    _check(lib, lib.janis_qk_rotate_norm_store(
        rows.data_ptr(), _DT[rows.dtype], rows.shape[1], T, H, G, d, int(rot), 1 if halves else 0,
        _t(inv_freq, "inv_freq", torch.float32, (max(rot // 2, 1),)) if rot else inv_freq.data_ptr(), 1 if unit_norm else 0,
        float(eps), _t(tok_pos, "tok_pos", torch.int32), _t(tok_seq, "tok_seq", torch.int32),
        _t(seq_slot, "seq_slot", torch.int32), kpool.data_ptr(), vpool.data_ptr() if vpool is not None else None,
        page_table.data_ptr(), page_table.shape[1], _stream()))
    return rows


HEAD_LINEAR_FEW_ROWS = 64        # up to here the kernel that keeps its rows in shared memory; above, in bfloat16, the library's batched product


def head_linear(x, x_head: int, x_off: int, w, out, o_head: int, o_off: int):
    """out[t, h * o_head + o_off + o] = sum_i w[h, o, i] x[t, h * x_head + x_off + i]: a product per head with a
    matrix of its own.  x [T, >= H x_head], w [H, O, I], out [T, >= H o_head], all of one dtype; float accumulation
    (in float32, and for few rows, in an order that depends on I alone)."""
    T = x.shape[0]
    Hn, O, I = w.shape
    _t(x, "x", _FLOATS, (T, None))
    _t(w, "w", x.dtype, (Hn, O, I))
    _t(out, "out", x.dtype, (T, None))
    if (Hn - 1) * x_head + x_off + I > x.shape[1] or (Hn - 1) * o_head + o_off + O > out.shape[1]:
        raise KernelError("head_linear: the heads do not fit the rows")
    if x.dtype == torch.bfloat16 and T > HEAD_LINEAR_FEW_ROWS:
        # many rows: the library's batched product (cuBLAS) over strided views, a batch entry per head, as
        # `linear_bf16` takes the library product for its large cases
        xv = x.as_strided((Hn, T, I), (x_head, x.stride(0), 1), x.storage_offset() + x_off)
        ov = out.as_strided((Hn, T, O), (o_head, out.stride(0), 1), out.storage_offset() + o_off)
        torch.bmm(xv, w.transpose(1, 2), out=ov)
        return out
    lib = mixers()
    _check(lib, lib.janis_head_linear(x.data_ptr(), _DT[x.dtype], x.shape[1], int(x_head), int(x_off), w.data_ptr(),
                                      out.data_ptr(), out.shape[1], int(o_head), int(o_off), T, Hn, I, O, _stream()))
    return out


def moe_route(z, correction, n_experts: int, group_count: int, group_keep: int, top: int, scale: float,
              shared_gate: bool, out, n_identity: int = 0, softmax: bool = False):
    """The router's weights per token and expert, 0 for experts that were not chosen: s = sigmoid(z), choice scores
    s + correction, the best group_keep of group_count groups (by the sum of a group's two largest choice scores), the
    `top` largest choice scores among their experts, w = s / (sum of the chosen s + 1e-20) * scale.  With
    shared_gate, column n_experts of z is a gate's logit and column n_experts of out its sigmoid.  z, out float32.
    softmax: s = softmax(z) over all entries instead.  n_identity: that many more entries behind the experts in z and
    correction (before the gate's column); they are scored and chosen like experts, and the weights of the chosen ones
    add up in one more column at the end of out."""
    T = z.shape[0]
    n = n_experts + n_identity
    cols_in = n + (1 if shared_gate else 0)
    cols_out = n_experts + (1 if shared_gate else 0) + (1 if n_identity else 0)
    lib = mixers()
    _check(lib, lib.janis_moe_route(_t(z, "z", torch.float32, (T, cols_in)), _t(correction, "correction", torch.float32, (n,)),
                                    T, n_experts, int(group_count), int(group_keep), int(top), float(scale),
                                    1 if shared_gate else 0, _t(out, "out", torch.float32, (T, cols_out)), int(n_identity),
                                    1 if softmax else 0, _stream()))
    return out


def moe_identity_add(out, y, wts, col: int):
    """out[t] += wts[t, col] y[t]: what a mixture's chosen identity entries add; out, y [T, W] of one dtype, wts float32."""
    T, W = out.shape
    lib = mixers()
    _check(lib, lib.janis_moe_identity_add(_t(out, "out", _FLOATS, (T, W)), _t(y, "y", out.dtype, (T, W)), _DT[out.dtype],
                                           _t(wts, "wts", torch.float32, (T, None)), wts.shape[1], int(col), T, W, _stream()))
    return out


def moe_expert_act(gu, wts, n_experts: int, ff: int, limit: float, shared_ff: int, shared_limit: float, alpha: float, out,
                   up_add: float = 1.0):
    """out[t, e * ff + j] = wts[t, e] * g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit,
    limit); gu [T, 2 (E ff + shared_ff)] holds each expert's ff gate columns followed by its ff up columns, the
    shared expert (weight wts[t, E], its own limit) last; out [T, E ff + shared_ff].  up_add replaces the 1 (0: the plain
    gated form); wts may have further columns behind the ones used."""
    T = gu.shape[0]
    total = n_experts * ff + shared_ff
    lib = mixers()
    _check(lib, lib.janis_moe_expert_act(_t(gu, "gu", _FLOATS, (T, 2 * total)), _DT[gu.dtype],
                                         _t(wts, "wts", torch.float32, (T, None)),
                                         n_experts, ff, float(limit), int(shared_ff), float(shared_limit), float(alpha),
                                         _t(out, "out", gu.dtype, (T, total)), T, wts.shape[1], float(up_add), _stream()))
    return out


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------

def argmax(logits, out):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_argmax(_t(logits, "logits", torch.float32), _t(out, "out", torch.int32, (R,)), R, V,
                                 _stream()))
    return out


def sample(logits, out, temp: float, top_p: float, seed: int, request_ids, token_index, u_out=None):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_sample(_t(logits, "logits", torch.float32), _t(out, "out", torch.int32, (R,)),
                                 _t(u_out, "u_out", torch.float32, (R,)) if u_out is not None else None, R, V,
                                 float(temp), float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF,
                                 _t(request_ids, "request_ids", torch.int32, (R,)),
                                 _t(token_index, "token_index", torch.int32, (R,)), _stream()))
    return out


def set_sample_kernel(which: int = 1) -> None:
    """Choose the kernel behind `sample`: 1 = the row's weights held in the shared memory of a cluster of up to 8
    CTAs (vocabularies up to about 368,000; the default), 0 = every pass over global memory (any vocabulary).
    For tests."""
    core().janis_set_sample_kernel(int(which))


def repeat_penalty(logits, recent, penalty: float):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_repeat_penalty(_t(logits, "logits", torch.float32), _t(recent, "recent", torch.int32, (R, None)),
                                         recent.shape[1], R, V, float(penalty), _stream()))
    return logits


def mask_tokens(logits, ids):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_mask_tokens(_t(logits, "logits", torch.float32), _t(ids, "ids", torch.int32), ids.numel(),
                                      R, V, _stream()))
    return logits
