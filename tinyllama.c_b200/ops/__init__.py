"""Tensor-level entry points of the CUDA kernels.

Each function checks devices, element types and strides, then calls one exported C
function of the kernel library on the current CUDA stream.  Nothing here computes on
the CPU or calls a library kernel: if the tensors are not on a GPU, or the library
cannot be built, the call raises.  Parts of the model call these through the module
(``ops.linear(...)``), which is also the seam a test uses to observe calls.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
PAGE = 64          # tokens per page of the key/value store (TLC_PAGE in tinyllama_c_b200.h)
# What the kernels are built for; a part checks its sizes against these when it is constructed, so that a
# configuration they do not cover is refused when the model is built, not at its first step.
MAX_HEAD_DIM = 256        # attention.cu: ATT_MAXD lanes-strided dims of a head (32 * 8)
MAX_STATE_SIZE = 256      # mamba.cu: state columns a warp keeps in registers (32 * 8)
MAX_CONV_TAPS = 17        # mamba.cu: CONV_MAX_TAPS + 1
MAX_HEADS = 65535         # a grid dimension
SSD_CHUNK = 128           # mamba_ssd.cu: rows of a chunk of the scan in matrix form

_vp, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
# Every function that csrc/tinyllama_c_b200.h declares: name -> (result, arguments).  A test parses the
# header and compares the kinds (pointer, int, float, long long), so that this table cannot drift from
# the definitions the compiler checked against the same header.
_SIGNATURES = {
    "tlc_last_error": (ctypes.c_char_p, []),
    "tlc_set_pdl": (None, [_i]),
    "tlc_linear_init": (_i, []),
    "tlc_attention_prefill_init": (_i, []),
    "tlc_ssd_init": (_i, []),
    "tlc_linear_error": (_i, []),
    "tlc_linear_error_clear": (None, []),
    "tlc_wait_limit_cycles": (_i, [_ll]),
    "tlc_selftest_bounded_wait": (_i, [_vp]),
    "tlc_embed": (_i, [_vp, _vp, _i, _i, _i, _i, _f, _vp, _vp]),
    "tlc_rmsnorm": (_i, [_vp, _i, _vp, _vp, _f, _i, _i, _vp, _i, _vp]),
    "tlc_layernorm": (_i, [_vp, _i, _vp, _vp, _vp, _f, _i, _i, _vp, _vp, _i, _vp]),
    "tlc_add_row": (_i, [_vp, _vp, _i, _i, _vp]),
    "tlc_difference_join": (_i, [_vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _f, _vp]),
    "tlc_gated_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _vp, _f, _i, _i, _i, _i, _vp, _i, _i, _f, _vp]),
    "tlc_swiglu": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _i, _vp]),
    "tlc_gather_rows": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "tlc_linear": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "tlc_linear_swiglu": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "tlc_linear_simt": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tlc_linear_skinny_ok": (_i, [_i, _i, _vp, _i, _i, _vp, _i, _i]),
    "tlc_linear_skinny": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tlc_linear_skinny_swiglu": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tlc_linear_tcgen05_ok": (_i, [_i, _i, _vp, _i, _i, _vp, _i]),
    "tlc_linear_tile_override": (None, [_i]),
    "tlc_linear_split_override": (None, [_i]),
    "tlc_linear_pair_override": (None, [_i]),
    "tlc_linear_skinny_pairs": (None, [_i]),
    "tlc_linear_tma_out": (None, [_i]),
    "tlc_linear_few_rows": (None, [_i]),
    "tlc_linear_few_rows_split": (None, [_i]),
    "tlc_linear_few_rows_min_tiles": (None, [_i]),
    "tlc_linear_few_rows_max_rows": (None, [_i]),
    "tlc_linear_few_rows_ok": (_i, [_i, _i, _vp, _i, _i, _vp, _i, _i, _i]),
    "tlc_linear_pairs": (_i, []),
    "tlc_rope_kv_store": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                               _i, _i, _vp]),
    "tlc_attention": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _f, _i, _i, _vp, _vp]),
    "tlc_attention_decode": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i,
                                  _i, _f, _i, _i, _vp, _vp]),
    "tlc_attention_decode_fused_ok": (_i, [_i, _i, _i]),
    "tlc_attention_decode_fused_passes": (_i, [_i]),
    "tlc_attention_decode_fused": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp,
                                        _vp, _i, _i, _i, _i, _f, _i, _i, _i, _f, _i, _i, _vp, _vp]),
    "tlc_attention_prefill_ok": (_i, [_i, _i]),
    "tlc_attention_prefill_chunks": (_i, [_i, _i, _i, _vp]),
    "tlc_attention_prefill": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp,
                                   _vp, _i, _i, _vp]),
    "tlc_attention_prefill_tc_ok": (_i, [_i, _i, _i, _i]),
    "tlc_attention_prefill_tc": (_i, [_vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i,
                                      _i, _i, _i, _i, _vp, _vp, _f, _i, _i, _vp, _vp]),
    "tlc_attention_prefill_tc_splits": (_i, [_i, _i, _i]),
    "tlc_mamba_conv": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i,
                            _i, _i, _i, _i, _i, _i, _vp]),
    "tlc_ssm_scan": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "tlc_ssm_scan_chunked": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i,
                                  _vp]),
    "tlc_ssd_ok": (_i, [_i, _i, _i, _i, _i]),
    "tlc_ssd_walk_override": (None, [_i]),
    "tlc_ssd_walk_blocks": (None, [_i]),
    "tlc_ssd_scratch_floats": (_ll, [_i, _i, _i, _i, _i, _i]),
    "tlc_ssm_scan_ssd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                              _i, _i, _vp, _vp]),
    "tlc_glu": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _i, _i, _f, _f, _vp]),
    "tlc_convert": (_i, [_vp, _i, _i, _i, _vp, _i, _i, _i, _vp]),
    "tlc_softcap": (_i, [_vp, _ll, _f, _vp]),
    "tlc_rmsnorm_mean_add": (_i, [_vp, _i, _vp, _f, _f, _vp, _f, _i, _i, _vp, _i, _vp, _i, _vp]),
    "tlc_qk_whole_norm": (_i, [_vp, _i, _i, _i, _vp, _i, _i, _vp, _f, _i, _vp]),
    "tlc_shift_mix": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "tlc_wkv_scan": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "tlc_moe_identity": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "tlc_rmsnorm_shift": (_i, [_vp, _vp, _vp, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "tlc_rmsnorm_add": (_i, [_vp, _i, _vp, _vp, _i, _i, _vp, _f, _i, _i, _vp, _i, _vp, _i, _vp]),
    "tlc_latent_prepare": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _f, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i,
                                _i, _i, _vp]),
    "tlc_latent_attention": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "tlc_latent_attention_tc_ok": (_i, [_i, _i, _i, _i]),
    "tlc_latent_attention_tc_splits": (_i, [_i, _i]),
    "tlc_latent_attention_tc_tile": (_i, [_i, _i, _i, _i]),
    "tlc_latent_attention_tc": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i,
                                     _vp]),
    "tlc_linear_heads": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "tlc_grouped_mma_ok": (_i, [_i, _i, _vp, _i, _i, _vp, _i]),
    "tlc_linear_heads_mma": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "tlc_moe_experts_mma": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, _i, _f, _f, _vp]),
    "tlc_mingru_scan": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _vp, _vp]),
    "tlc_moe_route": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _f, _vp]),
    "tlc_moe_gate_up": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _i, _i, _f, _f, _vp]),
    "tlc_qk_rotate_norm": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _f, _vp, _i, _vp, _vp, _f, _f, _vp]),
    "tlc_gate_mul": (_i, [_vp, _i, _i, _vp, _i, _i, _i, _i, _vp]),
    "tlc_delta_prepare": (_i, [_vp, _i, _i, _i, _i, _i, _f, _f, _vp, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp]),
    "tlc_delta_rule_split": (None, [_i]),
    "tlc_delta_rule": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _vp]),
    "tlc_moe_down": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "tlc_argmax": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "tlc_sample": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _f, _f, _f, _i, _f, _f, _vp, _vp]),
    "tlc_attention_decode_no_alloc": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i,
                                           _vp]),
}
_lib = None


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """Loads (building first if needed) the kernel library and declares its functions."""
    global _lib
    if _lib is None:
        lib = _build.load()
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
        if torch.cuda.is_available():                                     # before any stream capture
            for init in (lib.tlc_linear_init, lib.tlc_attention_prefill_init, lib.tlc_ssd_init):
                if init() != 0:
                    raise KernelError(f"kernel library set-up: {lib.tlc_last_error().decode()}")
        # Programmatic dependent launch for every kernel of the library, captured or not: a kernel's blocks are
        # scheduled (and fetch what does not depend on its predecessor) while the predecessor's last blocks finish.
        lib.tlc_set_pdl(1 if USE_PDL else 0)
    return _lib


USE_PDL = bool(int(os.environ.get("TLC_PDL", "1")))
_launches = 0


def launch_count() -> int:
    """How many kernel-launching library calls were made (captured calls count once at capture;
    a graph replay adds its calls through count_launches)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += int(n)


def _call(name: str, *args) -> None:
    global _launches
    lib = library()
    _launches += 1
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.tlc_last_error().decode()}")


# The current stream's handle is asked for by every call; torch.cuda.current_stream() builds a Stream object each
# time (several microseconds: a prompt step makes hundreds of calls and is bound by the host up to about 2,000
# tokens), torch's own raw query does not.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {dt}; the kernels take float32 and bfloat16")


def _gpu(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("tinyllama.c_b200 kernels run on a CUDA device only (got a CPU tensor); "
                              "there is no CPU path")


def _gpu_required() -> None:
    if not torch.cuda.is_available():
        raise KernelError("tinyllama.c_b200 kernels need a CUDA device; there is no CPU path")


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: expected a 2-D tensor with dense rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _out_rows(out: torch.Tensor, T: int, width: int, what: str) -> int:
    """Row stride of an output [T, width] whose rows are dense: the tensor itself, or a range of the
    columns of a wider buffer (several producers then fill one input of a following product)."""
    if tuple(out.shape) != (T, width):
        raise KernelError(f"{what}: output of shape {tuple(out.shape)}, expected {(T, width)}")
    return _rows(out, what + " output")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _f32vec(t: Optional[torch.Tensor], n: int, what: str) -> None:
    if t is None:
        return
    if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n:
        raise KernelError(f"{what}: expected {n} contiguous float32 values, got {tuple(t.shape)} {t.dtype}")


def _i32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what}: expected a contiguous int32 tensor, got {t.dtype}")


# ---- elementwise ---------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[t] = table[tokens[t]] * scale; out is float32 [T, D]."""
    _gpu(tokens, table, out)
    _i32(tokens, "embed tokens")
    T, (V, D) = tokens.numel(), table.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or tuple(out.shape) != (T, D) or not table.is_contiguous():
        raise KernelError("embed: out must be contiguous float32 [T, D] and the table contiguous")
    _call("tlc_embed", tokens.data_ptr(), table.data_ptr(), dtype_code(table.dtype), T, D, V, float(scale),
          out.data_ptr(), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x float32 [*, D] with dense rows (a range of the columns of a
    wider matrix will do)."""
    _gpu(x, weight, out, rows)
    D = x.shape[1]
    R = out.shape[0]
    if x.dtype != torch.float32 or not out.is_contiguous() or out.shape[1] != D:
        raise KernelError("rmsnorm: x must be float32 and out contiguous [R, D]")
    x_ld = _rows(x, "rmsnorm input")
    _f32vec(weight, D, "rmsnorm weight")
    if rows is not None:
        _i32(rows, "rmsnorm rows")
        if rows.numel() != R:
            raise KernelError("rmsnorm: one row index per output row")
    elif x.shape[0] != R:
        raise KernelError("rmsnorm: x and out differ in rows")
    _call("tlc_rmsnorm", x.data_ptr(), x_ld, _p(rows), weight.data_ptr(), float(eps), R, D, out.data_ptr(),
          dtype_code(out.dtype), _stream())


def gated_rmsnorm(y: torch.Tensor, z: torch.Tensor, weight: Optional[torch.Tensor], eps: float, n_groups: int,
                  norm_before_gate: bool, out: torch.Tensor, out_scale: float = 1.0,
                  y_add: Optional[torch.Tensor] = None, gate: str = "silu") -> None:
    """Gate y by silu(z) (or, gate "sigmoid", by sigmoid(z)) and RMS-normalise per group (either order); weight None = gate only.  The
    result is multiplied by out_scale; out [T, Di] may be a range of the columns of a wider buffer.
    y_add: a second summand of the input (the scan of prompts leaves its outputs as two), same shape as y."""
    _gpu(y, z, weight, out, y_add)
    T, Di = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous():
        raise KernelError("gated_rmsnorm: y must be contiguous float32 [T, Di]")
    if y_add is not None and (y_add.dtype != torch.float32 or not y_add.is_contiguous() or y_add.shape != y.shape):
        raise KernelError("gated_rmsnorm: y_add must be contiguous float32 of y's shape")
    out_ld = _out_rows(out, T, Di, "gated_rmsnorm")
    if z.shape != y.shape:
        raise KernelError("gated_rmsnorm: gate and input differ in shape")
    _f32vec(weight, Di, "gated_rmsnorm weight")
    _call("tlc_gated_rmsnorm", y.data_ptr(), _p(y_add), z.data_ptr(), dtype_code(z.dtype), _rows(z, "gate"), _p(weight),
          float(eps), T, Di, int(n_groups), int(bool(norm_before_gate)) | (2 if gate == "sigmoid" else 0), out.data_ptr(),
          dtype_code(out.dtype), out_ld, float(out_scale), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = silu(gate) * up, where gate_up holds gate | up as two halves, or (interleaved) in
    groups of 16 columns: 8 gates followed by their 8 ups."""
    _gpu(gate_up, out)
    T, F2 = gate_up.shape
    F = F2 // 2
    if not out.is_contiguous() or tuple(out.shape) != (T, F) or F2 != 2 * F:
        raise KernelError("swiglu: out must be contiguous [T, F]")
    if interleaved and F % 8:
        raise KernelError("swiglu: the interleaved layout needs a multiple of 8 features")
    _call("tlc_swiglu", gate_up.data_ptr(), dtype_code(gate_up.dtype), _rows(gate_up, "gate_up"), F, T,
          out.data_ptr(), dtype_code(out.dtype), int(bool(interleaved)), _stream())


GLU_ACTS = {"silu": 0, "gelu_tanh": 1}
DENSE_ACTS = dict(GLU_ACTS, swish_clamped=2)       # the clamped swish has no fused product epilogue: product, then glu()


def glu(gate_up: torch.Tensor, out: torch.Tensor, act: str = "silu", interleaved: bool = False, limit: float = 0.0,
        alpha: float = 1.0) -> None:
    """out = act(gate) * up with gate | up laid out as for swiglu; act: "silu", "gelu_tanh", or "swish_clamped": with
    g = min(gate, limit) and u = up held within +-limit, g * sigmoid(alpha * g) * (u + 1)."""
    _gpu(gate_up, out)
    T, F2 = gate_up.shape
    F = F2 // 2
    if act not in DENSE_ACTS:
        raise KernelError(f"glu: unknown activation '{act}'; known: {sorted(GLU_ACTS)}")
    if not out.is_contiguous() or tuple(out.shape) != (T, F) or F2 != 2 * F:
        raise KernelError("glu: out must be contiguous [T, F]")
    if interleaved and F % 8:
        raise KernelError("glu: the interleaved layout needs a multiple of 8 features")
    _call("tlc_glu", gate_up.data_ptr(), dtype_code(gate_up.dtype), _rows(gate_up, "gate_up"), F, T,
          out.data_ptr(), dtype_code(out.dtype), int(bool(interleaved)), DENSE_ACTS[act], float(limit), float(alpha), _stream())


CONVERT_ACTS = {"none": 0, "tanh": 1, "relu_squared": 2}


def convert(x: torch.Tensor, out: torch.Tensor, act: str = "none") -> None:
    """out = x (float32 [T, D], dense rows) in out's type, or with act "tanh" its tanh, with "relu_squared" max(x, 0)^2; out
    may be a range of the columns of a wider buffer."""
    _gpu(x, out)
    T, D = x.shape
    if x.dtype != torch.float32 or act not in CONVERT_ACTS:
        raise KernelError(f"convert: a float32 input; act one of {sorted(CONVERT_ACTS)}")
    _call("tlc_convert", x.data_ptr(), _rows(x, "convert input"), T, D, out.data_ptr(), dtype_code(out.dtype),
          _out_rows(out, T, D, "convert"), CONVERT_ACTS[act], _stream())


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None,
              weight2: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None) -> None:
    """out[r] = (x - mean(x)) / sqrt(var(x) + eps) * weight for x[rows[r]] or x[r] (float32 [*, D], dense rows), var the
    mean of the squared deviations; no bias.  weight2 and out2 (both or neither): the same normed rows times a second
    weight (two sublayers that each norm the same rows)."""
    _gpu(x, weight, out, rows, weight2, out2)
    D = x.shape[1]
    R = out.shape[0]
    if x.dtype != torch.float32 or not out.is_contiguous() or out.shape[1] != D:
        raise KernelError("layernorm: x must be float32 and out contiguous [R, D]")
    if (weight2 is None) != (out2 is None) or (out2 is not None and (not out2.is_contiguous() or out2.shape != out.shape
                                                                     or out2.dtype != out.dtype)):
        raise KernelError("layernorm: a second weight comes with a second output of the first one's shape and type")
    _f32vec(weight, D, "layernorm weight")
    _f32vec(weight2, D, "layernorm second weight")
    if rows is not None:
        _i32(rows, "layernorm rows")
        if rows.numel() != R:
            raise KernelError("layernorm: one row index per output row")
    elif x.shape[0] != R:
        raise KernelError("layernorm: x and out differ in rows")
    _call("tlc_layernorm", x.data_ptr(), _rows(x, "layernorm input"), _p(rows), weight.data_ptr(), _p(weight2), float(eps), R, D,
          out.data_ptr(), _p(out2), dtype_code(out.dtype), _stream())


def add_row(x: torch.Tensor, v: torch.Tensor) -> None:
    """x[t] += v for every row of x (contiguous float32 [T, D]); v float32 [D]."""
    _gpu(x, v)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2:
        raise KernelError("add_row: x must be contiguous float32 [T, D]")
    _f32vec(v, x.shape[1], "add_row vector")
    _call("tlc_add_row", x.data_ptr(), v.data_ptr(), x.shape[0], x.shape[1], _stream())


def difference_join(att: torch.Tensor, hd: int, out: torch.Tensor, hd_out: int, H: int, per_group: int, vd: int, lam: float,
                    eps: float, out_scale: float) -> None:
    """Two attention maps a query head: att [T, 2 * H * hd] holds virtual heads of hd values, the first map of head h (group
    g = h // per_group) at virtual head 2 g per_group + (h - g per_group), the second per_group heads further on;
    out[t, h * hd_out : + vd] = o / sqrt(mean(o^2) + eps) * out_scale with o = a1 - lam * a2 over the first vd values."""
    _gpu(att, out)
    T = att.shape[0]
    if att.dtype != out.dtype or att.shape[1] != 2 * H * hd:
        raise KernelError("difference_join: maps and result of one type, 2 * H heads of hd values in")
    _call("tlc_difference_join", att.data_ptr(), dtype_code(att.dtype), _rows(att, "attention maps"), int(hd), out.data_ptr(),
          _out_rows(out, T, H * hd_out, "difference_join"), int(hd_out), T, int(H), int(per_group), int(vd), float(lam), float(eps),
          float(out_scale), _stream())


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap), in place on a contiguous float32 tensor."""
    _gpu(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("softcap: a contiguous float32 tensor")
    _call("tlc_softcap", x.data_ptr(), x.numel(), float(cap), _stream())


def rmsnorm_mean_add(parts: torch.Tensor, weights: torch.Tensor, eps: float, scale: float, residual: torch.Tensor,
                     outer_weight: Optional[torch.Tensor] = None, outer_eps: float = 0.0, accumulate: bool = True,
                     copy: Optional[torch.Tensor] = None) -> None:
    """y = scale * sum_p rmsnorm(parts[:, p, :]) * weights[p]  (parts float32 [T, n, D], weights float32 [n, D]); then
    residual (+)= y, or with an outer weight [D] residual (+)= rmsnorm(y; outer_eps) * outer_weight.  copy [T, D] (float32
    or bfloat16, contiguous) receives the new residual rows as well."""
    _gpu(parts, weights, residual, outer_weight, copy)
    T, n, D = parts.shape
    if parts.dtype != torch.float32 or not parts.is_contiguous() or residual.dtype != torch.float32 \
            or not residual.is_contiguous() or tuple(residual.shape) != (T, D):
        raise KernelError("rmsnorm_mean_add: parts float32 [T, n, D] and residual float32 [T, D], contiguous")
    _f32vec(weights, n * D, "rmsnorm_mean_add weights")
    _f32vec(outer_weight, D, "rmsnorm_mean_add outer weight")
    _call("tlc_rmsnorm_mean_add", parts.data_ptr(), n, weights.data_ptr(), float(eps), float(scale), _p(outer_weight),
          float(outer_eps), T, D, residual.data_ptr(), int(bool(accumulate)), *_copy_of(copy, T, D, "rmsnorm_mean_add"), _stream())


def rmsnorm_shift(x: torch.Tensor, weight: torch.Tensor, mix: torch.Tensor, eps: float, state: torch.Tensor, step,
                  out: torch.Tensor) -> None:
    """n = rmsnorm(x) * weight; out[t] = n[t] + (n[t-1] - n[t]) * mix with n[t-1] the sequence's previous normed row:
    the row above, or the slot's row of state [n_slots, D] (zeros at position 0), which then receives the sequence's
    last normed row.  `step` is the StepInfo of the packed batch."""
    _gpu(x, weight, mix, state, out)
    T, D = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or tuple(out.shape) != (T, D):
        raise KernelError("rmsnorm_shift: x must be contiguous float32 [T, D] and out contiguous [T, D]")
    _f32vec(weight, D, "rmsnorm_shift weight")
    _f32vec(mix, D, "rmsnorm_shift mix")
    if state.dtype != torch.float32 or not state.is_contiguous() or state.shape[-1] != D or state.dim() != 2:
        raise KernelError("rmsnorm_shift: state must be contiguous float32 [n_slots, D]")
    _call("tlc_rmsnorm_shift", x.data_ptr(), weight.data_ptr(), mix.data_ptr(), float(eps), T, D, step.row_seq.data_ptr(),
          step.cu_seqlens.data_ptr(), step.slots.data_ptr(), step.start_pos.data_ptr(), state.data_ptr(), out.data_ptr(),
          dtype_code(out.dtype), _stream())


def rmsnorm_add(parts: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, residual: torch.Tensor,
                extra: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_sigmoid: bool = False,
                accumulate: bool = True, copy: Optional[torch.Tensor] = None) -> None:
    """residual[t] (+)= rmsnorm(y[t]) * weight (weight None: y[t] itself) with y[t] = sum_p parts[t, p, :] + g[t] *
    extra[t, :]; parts float32 [T, D] or [T, n, D], extra float32 [T, D], gate float32 [T] or one column of a wider
    float32 matrix; g is the gate, or its sigmoid.  copy [T, D] (float32 or bfloat16, contiguous) receives the new
    residual rows as well."""
    _gpu(parts, weight, residual, extra, gate, copy)
    T, D = residual.shape
    n = 0
    if parts is not None:
        n = 1 if parts.dim() == 2 else parts.shape[1]
        if parts.dtype != torch.float32 or not parts.is_contiguous() or parts.numel() != T * n * D:
            raise KernelError("rmsnorm_add: parts must be contiguous float32 [T, (n,) D]")
    if extra is not None and (extra.dtype != torch.float32 or not extra.is_contiguous() or tuple(extra.shape) != (T, D)):
        raise KernelError(f"rmsnorm_add: extra must be contiguous float32 {(T, D)}")
    gate_ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 1 or gate.numel() != T:
            raise KernelError("rmsnorm_add: gate must be float32 [T] (a column of a matrix will do)")
        gate_ld = gate.stride(0) if T > 1 else 1
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("rmsnorm_add: the residual stream must be contiguous float32")
    _f32vec(weight, D, "rmsnorm_add weight")
    _call("tlc_rmsnorm_add", _p(parts), n, _p(extra), _p(gate), int(gate_ld), int(bool(gate_sigmoid)), _p(weight), float(eps),
          T, D, residual.data_ptr(), int(bool(accumulate)), *_copy_of(copy, T, D, "rmsnorm_add"), _stream())


def _copy_of(copy: Optional[torch.Tensor], T: int, D: int, what: str):
    """Pointer and type code of the optional second output of the kernels that add into the residual stream."""
    if copy is None:
        return None, 0
    if tuple(copy.shape) != (T, D) or not copy.is_contiguous():
        raise KernelError(f"{what}: the copy must be contiguous {(T, D)}")
    return copy.data_ptr(), dtype_code(copy.dtype)


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _gpu(x, rows, out)
    _i32(rows, "gather rows")
    if x.dtype != torch.float32 or out.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("gather_rows: float32 contiguous tensors")
    _call("tlc_gather_rows", x.data_ptr(), rows.data_ptr(), rows.numel(), x.shape[1], out.data_ptr(), _stream())


# ---- linear -----------------------------------------------------------------------------
# Fewest rows for which bfloat16 products may go to the tiled tcgen05 kernel; with fewer rows
# (and, up to 64 rows, for narrow outputs) the weight matrix is streamed once by the mma.sync
# kernel.  TLC_TENSOR_CORE_MIN_ROWS overrides it (a huge value keeps the tiled kernel out).
TENSOR_CORE_MIN_ROWS = int(os.environ.get("TLC_TENSOR_CORE_MIN_ROWS", "33"))


def linear_split_override(splits: int) -> None:
    """Fixes how many blocks share the K-steps of a tile of the tensor-core product (0: chosen from the
    sizes, 1: none); for tests."""
    library().tlc_linear_split_override(int(splits))


def linear_pair_override(mode: int) -> None:
    """Pairs of blocks on 256 x 256 tiles in the tensor-core product: 0 where they pay, 1 never, 2 wherever
    the GPU can run them; for tests."""
    library().tlc_linear_pair_override(int(mode))


def linear_few_rows(on: bool, split: int = 0) -> None:
    """Whether products of 17..64 rows take the tensor-core kernel that puts the weights on the 128-row side and
    shares a tile's K-steps among the blocks of a cluster; split fixes the number of blocks per tile (1, 2, 4, 8;
    0: chosen from the sizes).  For tests and comparisons."""
    library().tlc_linear_few_rows(int(bool(on)))
    library().tlc_linear_few_rows_split(int(split))


def linear_tma_out(on: bool) -> None:
    """Whether 32-bit outputs of the tensor-core product leave through the copy engine (bulk tensor stores, and
    adds made at the L2 for sums into the output); for tests and comparisons."""
    library().tlc_linear_tma_out(int(bool(on)))


def linear_skinny_pairs(on: bool) -> None:
    """Whether the few-row product may give a tile of 16 columns to two blocks of a cluster, each with one half
    of K (it does where the matrix has fewer tiles than the GPU has SMs); for tests and comparisons."""
    library().tlc_linear_skinny_pairs(int(bool(on)))


def linear_pairs() -> int:
    """How many pairs of blocks (clusters of two) of the tensor-core product the GPU runs at once."""
    return int(library().tlc_linear_pairs())


def linear_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, colscale: Optional[torch.Tensor] = None,
                  colbias: Optional[torch.Tensor] = None, act: str = "silu") -> None:
    """out[M, F] = act(gate) * up with gate | up = (a w^T) * colscale + colbias, the 2F rows of w in
    groups of 16 (8 gate rows followed by their 8 up rows); act: "silu" or "gelu_tanh".  One kernel where the
    operands allow it (bfloat16, 16-byte aligned rows), else the product and the activation one after the other."""
    if act not in GLU_ACTS:
        raise KernelError(f"linear_swiglu: unknown activation '{act}'; known: {sorted(GLU_ACTS)}")
    _gpu(a, w, out, colscale, colbias)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or N % 16 or tuple(out.shape) != (M, N // 2) or not out.is_contiguous():
        raise KernelError(f"linear_swiglu: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    _f32vec(colscale, N, "linear colscale")
    _f32vec(colbias, N, "linear colbias")
    global _launches
    lib = library()
    _launches += 1
    rc = lib.tlc_linear_swiglu(a.data_ptr(), dtype_code(a.dtype), _rows(a, "linear input"), w.data_ptr(), dtype_code(w.dtype),
                               _rows(w, "linear weight"), out.data_ptr(), dtype_code(out.dtype), N // 2, _p(colscale),
                               _p(colbias), M, N, K, TENSOR_CORE_MIN_ROWS, GLU_ACTS[act], _stream())
    if rc == 1:                                   # no fused kernel for these operands
        _launches -= 1
        gu = torch.empty((M, N), dtype=torch.float32, device=a.device)
        linear(a, w, gu, colscale, colbias)
        glu(gu, out, act, interleaved=True)
    elif rc != 0:
        raise KernelError(f"tlc_linear_swiglu: {lib.tlc_last_error().decode()}")


def check_errors() -> None:
    """Raises if a tensor-core kernel gave up on a bounded wait (does not synchronise)."""
    code = library().tlc_linear_error()
    if code:
        library().tlc_linear_error_clear()
        raise KernelError(f"a kernel gave up on a bounded wait (code {code}: 1 loader, 2 issuer, 3 epilogue, 4 drain, "
                          f"5 accumulator of the tensor-core product; 9 the self-test); its output is incomplete")


def wait_limit_cycles(cycles: int) -> None:
    """How many clock cycles a bounded wait inside a kernel may spin before it gives up and reports
    (0: the default, about a second)."""
    lib = library()
    if lib.tlc_wait_limit_cycles(int(cycles)) != 0:
        raise KernelError(f"tlc_wait_limit_cycles: {lib.tlc_last_error().decode()}")


def selftest_bounded_wait() -> None:
    """Launches the error channel's self-test: a block waits on a barrier nobody arrives at, gives up at the
    limit and records code 9; check_errors() raises once the kernel has run."""
    _gpu_required()
    _call("tlc_selftest_bounded_wait", _stream())


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, colscale: Optional[torch.Tensor] = None,
           colbias: Optional[torch.Tensor] = None, accumulate: bool = False) -> None:
    """out[m, n] (+)= (sum_k a[m, k] w[n, k]) * colscale[n] + colbias[n].

    a [M, K] and out [M, N] may be row-strided views; w is [N, K].  Accumulation is
    32-bit.  float32 operands run on the CUDA cores in true 32-bit arithmetic."""
    _gpu(a, w, out, colscale, colbias)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"linear: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    _f32vec(colscale, N, "linear colscale")
    _f32vec(colbias, N, "linear colbias")
    _call("tlc_linear", a.data_ptr(), dtype_code(a.dtype), _rows(a, "linear input"), w.data_ptr(),
          dtype_code(w.dtype), _rows(w, "linear weight"), out.data_ptr(), dtype_code(out.dtype),
          _rows(out, "linear output"), _p(colscale), _p(colbias), int(bool(accumulate)), M, N, K,
          TENSOR_CORE_MIN_ROWS, _stream())


# ---- attention -------------------------------------------------------------------------------
DISABLE_TILED_ATTENTION = bool(int(os.environ.get("TLC_DISABLE_TILED_ATTENTION", "0")))
# Prompt attention on tcgen05 (0) or the mma.sync kernel everywhere (1); TLC_PROMPT_ATTENTION sets the start value,
# prompt_attention_override() changes it (tests run both).
_prompt_attention = int(os.environ.get("TLC_PROMPT_ATTENTION", "0"))


def prompt_attention_override(mode: int) -> None:
    """0: prompts of a bfloat16 cache with heads of 64 or 128 take the tcgen05 attention kernel; 1: the mma.sync one."""
    global _prompt_attention
    _prompt_attention = int(mode)


def rope_kv_store(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, k_pages: torch.Tensor,
                  v_pages: torch.Tensor, inv_freq: torch.Tensor, positions: torch.Tensor, row_seq: torch.Tensor,
                  slots: torch.Tensor, block_table: torch.Tensor, H: int, KV: int, hd: int,
                  write_kv: bool = True) -> None:
    """Rotates q and k at their absolute positions; writes q to q_out [T, H*hd] and k, v into
    the pages of their sequences ([page, KV, 64, hd])."""
    _gpu(qkv, q_out, k_pages, v_pages, inv_freq, positions, row_seq, slots, block_table)
    T = qkv.shape[0]
    for t, n in ((positions, "positions"), (row_seq, "row_seq"), (slots, "slots"), (block_table, "block_table")):
        _i32(t, n)
    if k_pages.dtype != q_out.dtype or v_pages.dtype != q_out.dtype:
        raise KernelError("rope_kv_store: q and the pages must share one element type")
    if not q_out.is_contiguous() or tuple(q_out.shape) != (T, H * hd) or not k_pages.is_contiguous() \
            or not v_pages.is_contiguous() or tuple(k_pages.shape[1:]) != (KV, PAGE, hd):
        raise KernelError("rope_kv_store: q_out must be contiguous [T, H*hd], pages contiguous [n, KV, 64, hd]")
    _f32vec(inv_freq, inv_freq.numel(), "rope inv_freq")
    _call("tlc_rope_kv_store", qkv.data_ptr(), dtype_code(qkv.dtype), dtype_code(q_out.dtype), _rows(qkv, "qkv"),
          q_off, k_off, v_off,
          q_out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), inv_freq.data_ptr(), 2 * inv_freq.numel(),
          positions.data_ptr(), row_seq.data_ptr(), slots.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          T, H, KV, hd, int(bool(write_kv)), _stream())


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
              positions: torch.Tensor, row_seq: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, H: int, KV: int,
              hd: int, scale: float, window: int = 0, decode_max_keys: int = 0,
              cu_seqlens: Optional[torch.Tensor] = None, start_pos: Optional[torch.Tensor] = None,
              max_keys: int = 0, max_blocks: int = 0, key_ranges: int = 0, softcap: float = 0.0, sink: bool = False,
              keep_first: int = 0, sink_values: Optional[torch.Tensor] = None) -> None:
    """Causal grouped-query attention of every row over its sequence's pages (keys 0..position,
    or the last `window` of them).  decode_max_keys > 0 says that the rows are single-token
    steps of sequences no longer than that: keys are then split across blocks.  With
    cu_seqlens and start_pos (rows of a sequence are consecutive positions from start_pos) the
    tiled tensor-core kernel serves bfloat16 heads of 64 or 128; with max_keys (the longest sequence
    after this step) it cuts the key range of long rows into pieces that run side by side.  max_blocks > 0
    bounds how many blocks (hence SMs) the tensor-core kernel of prompts holds at a time, for a caller that runs
    other kernels beside it; the result does not depend on it.  key_ranges > 0 fixes into how many ranges that
    kernel cuts the keys of a row tile (0: chosen: more than one for few rows over many keys).  softcap > 0: scores are
    softcap * tanh(score / softcap) after the scale; sink: the softmax's denominator has one more term of score 0, which
    carries no value (both served by the tcgen05 kernel of prompts, the warp kernels and the split-key kernels of single
    tokens).  sink_values float32 [H]: the sink's score per head instead of 0 (implies sink; the score is taken as it is, not
    scaled).  keep_first > 0 (with a window): the first keep_first keys of a sequence stay visible to every later query."""
    _gpu(q, k_pages, v_pages, block_table, positions, row_seq, slots, out, sink_values)
    T = q.shape[0]
    if sink_values is not None:
        _f32vec(sink_values, H, "attention sink scores")
        sink = True
    keep_first = int(keep_first) if window else 0
    if not q.is_contiguous() or tuple(q.shape) != (T, H * hd) or out.dtype != q.dtype or k_pages.dtype != q.dtype:
        raise KernelError("attention: q must be contiguous [T, H*hd], q and out of the pages' type")
    out_ld = _out_rows(out, T, H * hd, "attention")
    if decode_max_keys > 0 and H // KV <= 8:
        n_splits = (int(decode_max_keys) + 127) // 128
        part_o = torch.empty((T, H, n_splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, H, n_splits, 2), dtype=torch.float32, device=q.device)
        _call("tlc_attention_decode", q.data_ptr(), dtype_code(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), row_seq.data_ptr(),
              slots.data_ptr(), out.data_ptr(), part_o.data_ptr(), part_ml.data_ptr(), T, H, KV, hd, float(scale),
              int(window or 0), int(decode_max_keys), out_ld, float(softcap), int(bool(sink)), keep_first, _p(sink_values),
              _stream())
        return
    own_softmax = softcap > 0 or sink
    tiled = decode_max_keys <= 0 and cu_seqlens is not None and start_pos is not None and q.dtype == torch.bfloat16 \
        and hd in (64, 128) and not DISABLE_TILED_ATTENTION
    if tiled and _prompt_attention == 0 and max_keys > 0 and out_ld % 8 == 0 \
            and library().tlc_attention_prefill_tc_ok(BF16, hd, H, KV):
        B = slots.numel()
        # few row tiles and many keys (a piece of a long prompt): the keys in ranges that run side by side
        n_split = key_ranges if key_ranges > 0 else library().tlc_attention_prefill_tc_splits(T // 128 + B, H, int(max_keys))
        part_o = part_ml = None
        if n_split > 1:
            part_o = torch.empty((T, H, n_split, hd), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((T, H, n_split, 2), dtype=torch.float32, device=q.device)
        _call("tlc_attention_prefill_tc", q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
              block_table.data_ptr(), block_table.shape[1], cu_seqlens.data_ptr(), slots.data_ptr(), start_pos.data_ptr(),
              out.data_ptr(), B, T // 128 + B, H, KV, hd, float(scale), int(window or 0), int(max_keys), T,
              out_ld, int(max_blocks), int(n_split), _p(part_o), _p(part_ml), float(softcap), int(bool(sink)), keep_first,
              _p(sink_values), _stream())
        return
    if tiled and not own_softmax and keep_first == 0:
        B = slots.numel()
        n_tiles = T // 64 + B
        chunk = ctypes.c_int(0)
        n_chunks = library().tlc_attention_prefill_chunks(n_tiles, H, (int(max_keys) + 63) // 64, ctypes.byref(chunk)) \
            if max_keys > 0 else 1
        part_o = part_ml = None
        if n_chunks > 1:
            part_o = torch.empty((T, H, n_chunks, hd), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((T, H, n_chunks, 2), dtype=torch.float32, device=q.device)
        _call("tlc_attention_prefill", q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], cu_seqlens.data_ptr(), slots.data_ptr(), start_pos.data_ptr(), out.data_ptr(), B,
              n_tiles, H, KV, hd, float(scale), int(window or 0), (int(max_keys) + 63) // 64 if n_chunks > 1 else 0,
              row_seq.data_ptr(), _p(part_o), _p(part_ml), T, out_ld, _stream())
        return
    _call("tlc_attention", q.data_ptr(), dtype_code(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), row_seq.data_ptr(), slots.data_ptr(),
          out.data_ptr(), T, H, KV, hd, float(scale), int(window or 0), out_ld, float(softcap), int(bool(sink)), keep_first,
          _p(sink_values), _stream())


DISABLE_FUSED_DECODE_ATTENTION = bool(int(os.environ.get("TLC_DISABLE_FUSED_DECODE_ATTENTION", "0")))
FUSED_DECODE_COUNTERS = 65536      # arrival counters a caller of attention_decode_fused provides (rows x kv heads at most)


def new_arrival_counters(device) -> torch.Tensor:
    """Zeroed arrival counters for attention_decode_fused.  They belong to whoever launches the kernel (an
    attention mixer keeps its own): launches that share counters must not overlap on the GPU; every launch
    leaves them at zero.  Allocate them outside any stream capture."""
    return torch.zeros(FUSED_DECODE_COUNTERS, dtype=torch.int32, device=device)


def attention_decode_fused_ok(qkv: torch.Tensor, cache_dtype: torch.dtype, H: int, KV: int, hd: int) -> bool:
    """Whether attention_decode_fused takes this projection, cache type and these sizes."""
    return bool(qkv.is_cuda and qkv.dtype == torch.float32 and cache_dtype == torch.bfloat16
                and qkv.shape[0] * KV <= FUSED_DECODE_COUNTERS
                and not DISABLE_FUSED_DECODE_ATTENTION and library().tlc_attention_decode_fused_ok(H, KV, hd))


def attention_decode_fused(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, inv_freq: torch.Tensor, write_kv: bool, block_table: torch.Tensor,
                           positions: torch.Tensor, row_seq: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
                           H: int, KV: int, hd: int, scale: float, window: int, max_keys: int,
                           arrivals: torch.Tensor, softcap: float = 0.0, sink: bool = False, keep_first: int = 0,
                           sink_values: Optional[torch.Tensor] = None) -> None:
    """Single-token steps in one kernel: rotates the row's queries and new key (2 * len(inv_freq)
    leading dims of each head), stores the new key/value row into its page when write_kv, attends
    over the sequence's pages and writes out [T, H*hd] bfloat16.  qkv is float32 with dense rows.
    arrivals: the caller's counters (new_arrival_counters).  softcap, sink, keep_first and sink_values as in attention()."""
    _gpu(qkv, k_pages, v_pages, inv_freq, block_table, positions, row_seq, slots, out, sink_values)
    if sink_values is not None:
        _f32vec(sink_values, H, "attention sink scores")
        sink = True
    T = qkv.shape[0]
    for t, n in ((positions, "positions"), (row_seq, "row_seq"), (slots, "slots"), (block_table, "block_table")):
        _i32(t, n)
    if qkv.dtype != torch.float32 or k_pages.dtype != torch.bfloat16 or v_pages.dtype != torch.bfloat16 \
            or out.dtype != torch.bfloat16:
        raise KernelError("attention_decode_fused: float32 projections, bfloat16 pages and output")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[1:]) != (KV, PAGE, hd) \
            or v_pages.shape != k_pages.shape:
        raise KernelError("attention_decode_fused: pages must be contiguous [n, KV, 64, hd]")
    out_ld = _out_rows(out, T, H * hd, "attention_decode_fused")
    ld = _rows(qkv, "qkv")
    if max(q_off + H * hd, k_off + KV * hd, v_off + KV * hd) > max(ld, qkv.shape[1]):
        raise KernelError("attention_decode_fused: q, k or v lies outside the projection's row")
    _f32vec(inv_freq, inv_freq.numel(), "rope inv_freq")
    n_splits = (int(max_keys) + 127) // 128
    part_o = torch.empty((T, H, n_splits, hd), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((T, H, n_splits, 2), dtype=torch.float32, device=qkv.device)
    _gpu(arrivals)
    _i32(arrivals, "arrival counters")
    if arrivals.numel() < T * KV:
        raise KernelError(f"attention_decode_fused: {T * KV} (row, kv head) pairs need as many arrival counters, "
                          f"{arrivals.numel()} given")
    _call("tlc_attention_decode_fused", qkv.data_ptr(), ld, q_off, k_off, v_off, k_pages.data_ptr(), v_pages.data_ptr(),
          inv_freq.data_ptr(), 2 * inv_freq.numel(), int(bool(write_kv)), block_table.data_ptr(), block_table.shape[1],
          positions.data_ptr(), row_seq.data_ptr(), slots.data_ptr(), out.data_ptr(), part_o.data_ptr(),
          part_ml.data_ptr(), arrivals.data_ptr(), T, H, KV, hd, float(scale), int(window or 0), int(max_keys), out_ld,
          float(softcap), int(bool(sink)), int(keep_first) if window else 0, _p(sink_values), _stream())


def attention_decode_fused_passes(passes: int) -> None:
    """Fixes how many rounds of chunks a block of the fused single-token attention takes one after the
    other (0: chosen from the grid); for tests of the running statistics."""
    library().tlc_attention_decode_fused_passes(int(passes))


DISABLE_SSD = bool(int(os.environ.get("TLC_DISABLE_SSD", "0")))


# ---- Mamba2 -------------------------------------------------------------------------------------
def mamba_conv(proj: torch.Tensor, xbc_off: int, dt_off: int, w: torch.Tensor, bias: Optional[torch.Tensor],
               dt_bias: torch.Tensor, A: torch.Tensor, conv_state: torch.Tensor, cu_seqlens: torch.Tensor,
               row_seq: torch.Tensor, slots: torch.Tensor, start_pos: torch.Tensor, xbc_out: torch.Tensor,
               dt_out: torch.Tensor, dA_out: torch.Tensor, single_rows: bool = False, bf16_run: bool = False,
               all_fresh: bool = False) -> None:
    """Causal depthwise convolution + SiLU of the xBC columns of proj, continuing each
    sequence's window (conv_state [n_slots, K-1, Cd], updated in place); also
    dt = softplus(dt + dt_bias) and dA = exp(dt * A) per row and head.  single_rows says
    that every sequence brings exactly one row (row b belongs to sequence b); bf16_run says that the
    model computes in bfloat16: x|B|C, operands of the scan's matrix products, are then rounded to
    bfloat16 values whatever type they are stored in, and the SiLU of prompts takes the fast exponential
    and reciprocal.  xbc_out is float32, or
    bfloat16 where the scan that follows takes its operands in that type (ssm_scan with A).  all_fresh says that
    every sequence of the step starts at position 0 (the caller knows the start positions on the host): no stored
    window is read then, and the convolution's own kernel leaves the new windows (one launch less)."""
    _gpu(proj, w, bias, dt_bias, A, conv_state, cu_seqlens, row_seq, slots, start_pos, xbc_out, dt_out, dA_out)
    T = proj.shape[0]
    Cd, K = w.shape
    Hs = dt_bias.numel()
    B = slots.numel()
    _f32vec(w, Cd * K, "conv weight")
    _f32vec(bias, Cd, "conv bias")
    _f32vec(dt_bias, Hs, "dt_bias")
    _f32vec(A, Hs, "A")
    for t, n in ((cu_seqlens, "cu_seqlens"), (row_seq, "row_seq"), (slots, "slots"), (start_pos, "start_pos")):
        _i32(t, n)
    if conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or tuple(conv_state.shape[1:]) != (K - 1, Cd):
        raise KernelError("mamba_conv: conv_state must be contiguous float32 [n_slots, K-1, Cd]")
    for t, shp, n in ((dt_out, (T, Hs), "dt_out"), (dA_out, (T, Hs), "dA_out")):
        if t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != shp:
            raise KernelError(f"mamba_conv: {n} must be contiguous float32 {shp}")
    if not xbc_out.is_contiguous() or tuple(xbc_out.shape) != (T, Cd):
        raise KernelError(f"mamba_conv: xbc_out must be contiguous {(T, Cd)}")
    _call("tlc_mamba_conv", proj.data_ptr(), dtype_code(proj.dtype), _rows(proj, "proj"), xbc_off, dt_off,
          w.data_ptr(), _p(bias), dt_bias.data_ptr(), A.data_ptr(), conv_state.data_ptr(), cu_seqlens.data_ptr(),
          row_seq.data_ptr(), slots.data_ptr(), start_pos.data_ptr(), xbc_out.data_ptr(), dtype_code(xbc_out.dtype),
          dt_out.data_ptr(), dA_out.data_ptr(), T, B, Cd, K, Hs, int(bool(single_rows)), int(bool(bf16_run)),
          int(bool(all_fresh)), _stream())


def ssd_walk_blocks(blocks: int) -> None:
    """How many blocks of the tcgen05 walk work through the (sequence, head, rows) items (0: one an SM at most);
    for tests: with few blocks each walks many sequences in turn."""
    library().tlc_ssd_walk_blocks(int(blocks))


def ssd_walk_override(mode: int) -> None:
    """Which kernel walks a sequence's chunks where both are built (0: tcgen05 with the state in tensor memory for
    states of 128 or 256 columns; 1: always mma.sync with the state in registers); for tests."""
    library().tlc_ssd_walk_override(int(mode))


def ssd_ok(Hs: int, P: int, N: int, G: int) -> bool:
    """Whether the scan of prompts in matrix form (bfloat16 operands, ssm_scan with A) is built for these sizes."""
    return bool(not DISABLE_SSD and library().tlc_ssd_ok(Hs, P, N, G, Hs * P + 2 * G * N))


_aux_streams: dict = {}


def _aux_stream(device) -> "torch.cuda.Stream":
    """A second stream per device and current stream, for work that runs beside a kernel chain of the current one."""
    key = (torch.device(device).index, _stream())        # (the raw handle: torch.cuda.current_stream() costs 10 us)
    if key not in _aux_streams:
        if len(_aux_streams) > 64:
            _aux_streams.clear()
        _aux_streams[key] = torch.cuda.Stream(device=device)
    return _aux_streams[key]


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, dA: torch.Tensor, Dskip: torch.Tensor, state: torch.Tensor,
             cu_seqlens: torch.Tensor, slots: torch.Tensor, start_pos: torch.Tensor, y: torch.Tensor, Hs: int, P: int,
             N: int, G: int, chunks=None, A: Optional[torch.Tensor] = None, y_part: Optional[torch.Tensor] = None) -> bool:
    """Selective scan of every sequence in order, from its slot's state (zero at position 0);
    state [n_slots, Hs, P, N] float32 is updated in place; y [T, Hs*P] float32 is before gating.
    chunks = (seg_start [n+1], seg_seq [n], seq_seg_start [B+1]) cuts the sequences into
    chunks that run in parallel (same result up to rounding).  With a bfloat16 xbc and A (the per-head
    decay rate, dA = exp(dt * A)) the chunks, of at most 128 rows, run in matrix form on the tensor cores
    with bfloat16 operands (see ssd_ok for the sizes); every 32-bit run passes a float32 xbc.
    y_part (float32, y's shape; matrix form only): the outputs may then come as two summands, what needs no state in
    y_part (computed on a second stream beside the walk over the chunks) and the state's share in y; returns True
    if they did (the caller adds them), False if y holds the outputs."""
    _gpu(xbc, dt, dA, Dskip, state, cu_seqlens, slots, start_pos, y, y_part)
    T, Cd = xbc.shape
    if Cd != Hs * P + 2 * G * N:
        raise KernelError("ssm_scan: xbc width does not match Hs*P + 2*G*N")
    matrix_form = xbc.dtype == torch.bfloat16
    for t, shp, n in ((xbc, (T, Cd), "xbc"), (dt, (T, Hs), "dt"), (dA, (T, Hs), "dA"), (y, (T, Hs * P), "y")):
        want = torch.bfloat16 if (n == "xbc" and matrix_form) else torch.float32
        if t.dtype != want or not t.is_contiguous() or tuple(t.shape) != shp:
            raise KernelError(f"ssm_scan: {n} must be contiguous {want} {shp}")
    _f32vec(Dskip, Hs, "D")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (Hs, P, N):
        raise KernelError("ssm_scan: state must be contiguous float32 [n_slots, Hs, P, N]")
    if matrix_form and (chunks is None or A is None or not ssd_ok(Hs, P, N, G)):
        raise KernelError("ssm_scan: a bfloat16 x|B|C is for the chunked scan in matrix form (chunks, A, sizes of ssd_ok)")
    if chunks is not None:
        seg_start, seg_seq, seq_seg_start = chunks
        for t, n in ((seg_start, "seg_start"), (seg_seq, "seg_seq"), (seq_seg_start, "seq_seg_start")):
            _gpu(t)
            _i32(t, n)
        n_seg = seg_seq.numel()
        lib = library()
        if matrix_form:
            _f32vec(A, Hs, "A")
            scratch = torch.empty(lib.tlc_ssd_scratch_floats(n_seg, T, Hs, P, N, G), dtype=torch.float32, device=xbc.device)
            if y_part is not None and (y_part.dtype != torch.float32 or not y_part.is_contiguous() or y_part.shape != y.shape):
                raise KernelError("ssm_scan: y_part must be contiguous float32 of y's shape")
            used = ctypes.c_int(0)
            aux = _aux_stream(xbc.device).cuda_stream if y_part is not None and not torch.cuda.is_current_stream_capturing() else None
            _call("tlc_ssm_scan_ssd", xbc.data_ptr(), dt.data_ptr(), A.data_ptr(), Dskip.data_ptr(), state.data_ptr(),
                  scratch.data_ptr(), seg_start.data_ptr(), seg_seq.data_ptr(), seq_seg_start.data_ptr(),
                  slots.data_ptr(), start_pos.data_ptr(), y.data_ptr(), _p(y_part), ctypes.byref(used), slots.numel(), n_seg,
                  T, Hs, P, N, G, Cd, _stream(), aux)
            return bool(used.value)
        scratch = torch.empty(n_seg * Hs * (P * N + 1), dtype=torch.float32, device=xbc.device)
        _call("tlc_ssm_scan_chunked", xbc.data_ptr(), dt.data_ptr(), dA.data_ptr(), Dskip.data_ptr(), state.data_ptr(),
              scratch.data_ptr(), seg_start.data_ptr(), seg_seq.data_ptr(), seq_seg_start.data_ptr(), slots.data_ptr(),
              start_pos.data_ptr(), y.data_ptr(), slots.numel(), n_seg, Hs, P, N, G, Cd, _stream())
        return False
    _call("tlc_ssm_scan", xbc.data_ptr(), dt.data_ptr(), dA.data_ptr(), Dskip.data_ptr(), state.data_ptr(),
          cu_seqlens.data_ptr(), slots.data_ptr(), start_pos.data_ptr(), y.data_ptr(), slots.numel(), Hs, P, N, G, Cd,
          _stream())
    return False


# ---- sampling -------------------------------------------------------------------------------------
def new_argmax_work(rows: int, device) -> torch.Tensor:
    """Zeroed workspace for argmax over `rows` rows (every launch leaves it zero); its owner's launches must not
    overlap on the GPU.  Allocate it outside any stream capture."""
    return torch.zeros(2 * max(1, int(rows)), dtype=torch.int64, device=device)


def argmax(logits: torch.Tensor, out: torch.Tensor, work: Optional[torch.Tensor] = None) -> None:
    """out[r] = first index of the maximum of logits[r].  With `work` (new_argmax_work) a row is spread over
    many blocks; without, one block takes a row."""
    _gpu(logits, out, work)
    _i32(out, "argmax out")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("argmax: logits must be contiguous float32")
    if work is not None and (work.dtype != torch.int64 or not work.is_contiguous() or work.numel() < 2 * logits.shape[0]):
        raise KernelError("argmax: work must be a contiguous int64 tensor of at least 2 values per row")
    _call("tlc_argmax", logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(), _p(work), _stream())


def sample(logits: torch.Tensor, work: torch.Tensor, history: Optional[torch.Tensor], uniforms: torch.Tensor,
           temperature: float, top_k: int, top_p: float, min_p: float, repeat_penalty: float,
           frequency_penalty: float, presence_penalty: float, out: torch.Tensor) -> None:
    """One token per row from penalised, temperature-scaled, top-k / min-p / top-p filtered
    logits; `history` [R, n] int32 (-1 = empty) is the penalty window, `uniforms` [R] the draws,
    `work` a [R, V] float32 scratch."""
    _gpu(logits, work, history, uniforms, out)
    R, V = logits.shape
    _i32(out, "sample out")
    if logits.dtype != torch.float32 or not logits.is_contiguous() or work.dtype != torch.float32 \
            or not work.is_contiguous() or work.numel() < R * V:
        raise KernelError("sample: logits and work must be contiguous float32 [R, V]")
    _f32vec(uniforms, R, "sample uniforms")
    n_hist = 0
    if history is not None:
        _i32(history, "sample history")
        n_hist = history.shape[1]
    _call("tlc_sample", logits.data_ptr(), work.data_ptr(), _p(history), uniforms.data_ptr(), R, V,
          float(temperature), int(top_k), float(top_p), float(min_p), float(repeat_penalty), n_hist,
          float(frequency_penalty), float(presence_penalty), out.data_ptr(), _stream())


# ---- attention over a shared latent -------------------------------------------------------------------
MAX_LATENT = 512          # latent_attention.cu: 32 * LAT_MAXV values of a latent


def latent_prepare(proj: Optional[torch.Tensor], q_off: int, dkv_off: Optional[int], norm_weight: Optional[torch.Tensor], eps: float,
                   inv_freq: torch.Tensor, step, block_table: torch.Tensor, pages: torch.Tensor, qn: torch.Tensor,
                   qa: torch.Tensor, H: int, dn: int, r: int, R: int, q_proj: Optional[torch.Tensor] = None) -> None:
    """From a row's projections (float32 [T, *]: H heads of (dn | r) query values at q_off, R + r down-projected values
    at dkv_off, None for a layer that reads another layer's rows; q_proj: the buffer that holds the queries, where it
    is not proj itself, which may then be None with dkv_off None): the unrotated query parts to qn [T, H*dn], the
    rotated ones into the last r columns of every head of qa [T, H*(R+r)], and the cache row [rmsnorm(c) * norm_weight
    | rotated kr] into its page of pages [n, 64, R+r].  The rotation turns interleaved pairs of the first
    2 * len(inv_freq) dimensions."""
    if q_proj is None:
        q_proj = proj
    if proj is None:
        if dkv_off is not None:
            raise KernelError("latent_prepare: a down-projection's columns without its buffer")
        proj = q_proj
    _gpu(proj, q_proj, norm_weight, inv_freq, block_table, pages, qn, qa)
    T = q_proj.shape[0]
    _i32(block_table, "block_table")
    if proj.dtype != torch.float32 or q_proj.dtype != torch.float32 or proj.shape[0] != T:
        raise KernelError("latent_prepare: float32 projections of equal rows")
    if qn.dtype != pages.dtype or qa.dtype != pages.dtype or not qn.is_contiguous() or not qa.is_contiguous() \
            or tuple(qn.shape) != (T, H * dn) or tuple(qa.shape) != (T, H * (R + r)):
        raise KernelError("latent_prepare: qn [T, H*dn] and qa [T, H*(R+r)] must be contiguous and of the pages' type")
    if not pages.is_contiguous() or tuple(pages.shape[1:]) != (PAGE, R + r):
        raise KernelError("latent_prepare: pages must be contiguous [n, 64, R+r]")
    if dkv_off is not None:
        _f32vec(norm_weight, R, "latent norm weight")
    _f32vec(inv_freq, inv_freq.numel(), "rotation inv_freq")
    _call("tlc_latent_prepare", q_proj.data_ptr(), _rows(q_proj, "q_proj"), int(q_off), proj.data_ptr(), _rows(proj, "proj"),
          -1 if dkv_off is None else int(dkv_off),
          _p(norm_weight), float(eps), inv_freq.data_ptr(), 2 * inv_freq.numel(), step.positions.data_ptr(),
          step.row_seq.data_ptr(), step.slots.data_ptr(), block_table.data_ptr(), block_table.shape[1], pages.data_ptr(),
          qn.data_ptr(), qa.data_ptr(), dtype_code(pages.dtype), T, H, dn, r, R, _stream())


_latent_tc = not bool(int(os.environ.get("TLC_DISABLE_LATENT_TC", "0")))


def latent_attention_tc(on: bool) -> None:
    """Whether bfloat16 latent attention takes the tensor-core kernel where it is built (TLC_DISABLE_LATENT_TC=1 sets the
    start value to off); for tests and comparisons."""
    global _latent_tc
    _latent_tc = bool(on)


def latent_attention(qa: torch.Tensor, pages: torch.Tensor, sink: Optional[torch.Tensor], block_table: torch.Tensor, step,
                     out: torch.Tensor, H: int, R: int, r: int, scale: float, key_ranges: int = 0, window: int = 0) -> None:
    """out [T, H*R]: every head's softmax-weighted sum of the latents of keys 0..position (with window > 0: of the last
    `window` of them), scores (qa . [c | kr]) * scale, with the head's sink (None: no sink) in the denominator.  bfloat16 rows of sizes the tensor-core kernel is built for take it (all
    heads of a row share every page read); key_ranges > 0 fixes into how many ranges it cuts a tile's keys (0: chosen:
    more than one for few rows over many keys)."""
    _gpu(qa, pages, sink, block_table, out)
    T = qa.shape[0]
    _i32(block_table, "block_table")
    _f32vec(sink, H, "attention sink")
    if qa.dtype != pages.dtype or out.dtype != pages.dtype or not qa.is_contiguous() or not out.is_contiguous() \
            or tuple(qa.shape) != (T, H * (R + r)) or tuple(out.shape) != (T, H * R) or not pages.is_contiguous():
        raise KernelError("latent_attention: qa [T, H*(R+r)] and out [T, H*R] contiguous and of the pages' type")
    lib = library()
    if _latent_tc and lib.tlc_latent_attention_tc_ok(dtype_code(pages.dtype), H, R, r):
        hp = 1
        while hp < H and hp < 64:
            hp *= 2
        B = step.n_seqs
        pairs = lib.tlc_latent_attention_tc_tile(T, B, R, r)          # (row, head) pairs a tile: 128 for prompts, else 64
        n_tiles = T // (pairs // hp) + B
        seen = int(step.max_context) if not window else min(int(step.max_context), int(window) + pairs // hp)   # keys a tile sees
        n_split = min(64, key_ranges) if key_ranges > 0 else lib.tlc_latent_attention_tc_splits(n_tiles * ((H + hp - 1) // hp), seen)
        part_o = part_ml = None
        if n_split > 1:
            part_o = torch.empty((T, H, n_split, R), dtype=torch.float32, device=qa.device)
            part_ml = torch.empty((T, H, n_split, 2), dtype=torch.float32, device=qa.device)
        _call("tlc_latent_attention_tc", qa.data_ptr(), pages.data_ptr(), _p(sink), block_table.data_ptr(),
              block_table.shape[1], step.cu_seqlens.data_ptr(), step.slots.data_ptr(), step.start_pos.data_ptr(),
              out.data_ptr(), _p(part_o), _p(part_ml), B, T, pairs, n_tiles, H, R, r, float(scale), int(n_split), int(window or 0),
              _stream())
        return
    _call("tlc_latent_attention", qa.data_ptr(), pages.data_ptr(), dtype_code(pages.dtype), _p(sink),
          block_table.data_ptr(), block_table.shape[1], step.positions.data_ptr(), step.row_seq.data_ptr(),
          step.slots.data_ptr(), out.data_ptr(), T, H, R, r, float(scale), int(window or 0), _stream())


_grouped_mma = not bool(int(os.environ.get("TLC_DISABLE_GROUPED_MMA", "0")))


def grouped_mma(on: bool) -> None:
    """Whether bfloat16 products per head and per expert take the mma.sync kernel where their operands are aligned for it
    (TLC_DISABLE_GROUPED_MMA=1 sets the start value to off); for tests and comparisons."""
    global _grouped_mma
    _grouped_mma = bool(on)


def linear_heads(a: torch.Tensor, a_head_stride: int, w: torch.Tensor, out: torch.Tensor, o_head_stride: int) -> None:
    """out[t, h, n] = sum_k a[t, h, k] w[h, n, k]: w [H, N, K] contiguous; a and out are 2-D with dense rows, head h of a
    row starting a_head_stride * h (o_head_stride * h) elements in."""
    _gpu(a, w, out)
    H, N, K = w.shape
    T = a.shape[0]
    if not w.is_contiguous() or out.shape[0] != T:
        raise KernelError("linear_heads: w must be contiguous [H, N, K], a and out of equal rows")
    lda, ldo = _rows(a, "linear_heads input"), _rows(out, "linear_heads output")
    if (H - 1) * a_head_stride + K > max(lda, a.shape[1]) or (H - 1) * o_head_stride + N > max(ldo, out.shape[1]):
        raise KernelError("linear_heads: a head lies outside its row")
    if _grouped_mma and library().tlc_grouped_mma_ok(dtype_code(a.dtype), dtype_code(w.dtype), a.data_ptr(), lda, int(a_head_stride),
                                                     w.data_ptr(), K):
        _call("tlc_linear_heads_mma", a.data_ptr(), lda, int(a_head_stride), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), ldo,
              int(o_head_stride), T, H, N, K, _stream())
        return
    _call("tlc_linear_heads", a.data_ptr(), dtype_code(a.dtype), lda, int(a_head_stride), w.data_ptr(), dtype_code(w.dtype),
          out.data_ptr(), dtype_code(out.dtype), ldo, int(o_head_stride), T, H, N, K, _stream())


# ---- minGRU ------------------------------------------------------------------------------------------------
def mingru_scan(proj: torch.Tensor, z_off: int, u_off: int, g_off: int, width: int, state: torch.Tensor, step,
                out: torch.Tensor, chunks=None) -> None:
    """The gated recurrence S <- (1 - z) S + z cand of every sequence from its slot's state [n_slots, W] (zero at
    position 0; updated in place), out[t] = S * silu(g); z, u, g are column ranges of proj (float32).  chunks: the
    step's chunk table (seg_start, seg_seq, seq_seg_start) or None for the row-by-row form."""
    _gpu(proj, state, out)
    T = proj.shape[0]
    if proj.dtype != torch.float32 or state.dtype != torch.float32 or not state.is_contiguous() or state.shape[-1] != width:
        raise KernelError("mingru_scan: float32 projections and a contiguous float32 state [n_slots, W]")
    out_ld = _out_rows(out, T, width, "mingru_scan")
    seg = seq_seg = scratch = None
    n_seg = 0
    if chunks is not None:
        seg, _, seq_seg = chunks
        n_seg = seg.numel() - 1
        scratch = torch.empty(2 * n_seg * width, dtype=torch.float32, device=proj.device)
    _call("tlc_mingru_scan", proj.data_ptr(), _rows(proj, "proj"), int(z_off), int(u_off), int(g_off), int(width),
          state.data_ptr(), step.cu_seqlens.data_ptr(), step.slots.data_ptr(), step.start_pos.data_ptr(), step.n_seqs,
          out.data_ptr(), dtype_code(out.dtype), out_ld, _p(seg), _p(seq_seg), n_seg, _p(scratch), _stream())


# ---- mixture of experts ------------------------------------------------------------------------------------
def _moe_mma_ok(x: torch.Tensor, w_gate_up: torch.Tensor, act_dtype: torch.dtype, F: Optional[int] = None) -> bool:
    D = w_gate_up.shape[2]
    F = w_gate_up.shape[1] // 2 if F is None else F
    return bool(_grouped_mma and act_dtype == torch.bfloat16 and F % 8 == 0 and D % 8 == 0
                and library().tlc_grouped_mma_ok(dtype_code(x.dtype), dtype_code(w_gate_up.dtype), x.data_ptr(), _rows(x, "moe input"),
                                                 0, w_gate_up.data_ptr(), D))


def moe_tile_rows(x: torch.Tensor, w_gate_up: torch.Tensor, act_dtype: torch.dtype, top: int, F: Optional[int] = None) -> int:
    """Rows of a tile of the experts' products for this input: 64 where the tensor-core kernel runs and an expert gets
    64 rows or more on average, else 32.  The routing is made for that number (moe_route) and carries it."""
    E = w_gate_up.shape[0]
    return 64 if _moe_mma_ok(x, w_gate_up, act_dtype, F) and x.shape[0] * top >= 64 * E else 32


ROUTE_WEIGHTS = {"sigmoid": 0, "softmax": 1, "softmax_all": 2}
MOE_ACTS = dict(GLU_ACTS, swish_clamped=2, relu_squared=3)
UNGATED_ACTS = ("relu_squared",)          # experts of one product: w_up [E, F, D], no gate


def moe_route(logits: torch.Tensor, n_experts: int, top: int, tile_rows: int = 32, weights: str = "sigmoid",
              choice_bias: Optional[torch.Tensor] = None, n_identity: int = 0, sum_to: float = 0.0):
    """Routing of every row of logits (float32 [T, >= E], the first E columns): returns (ids [T*top] int32, weights
    [T*top] float32 = sigmoid of the chosen logits, or with weights "softmax" a softmax restricted to the picked logits,
    order [T*top], offsets [E+1], tile_off [E+1], tile_rows) as tlc_moe_route describes them.  With weights "softmax_all"
    the scores are the softmax over all n_experts outputs, an expert is chosen by score + choice_bias and weighted by its
    score.  The last n_identity of the n_experts outputs have no weights of an expert: no tile covers their pairs.  sum_to > 0
    (weights "softmax_all"): a token's weights are divided by their sum (+ 1e-20) and multiplied by sum_to."""
    if sum_to and weights != "softmax_all":
        raise KernelError("moe_route: weights normed to a sum go with weights 'softmax_all'")
    if weights not in ROUTE_WEIGHTS:
        raise KernelError(f"moe_route: unknown weighting '{weights}'; known: {sorted(ROUTE_WEIGHTS)}")
    _gpu(logits)
    T = logits.shape[0]
    if logits.dtype != torch.float32 or logits.shape[1] < n_experts:
        raise KernelError("moe_route: float32 logits [T, >= E]")
    dev = logits.device
    ints = torch.empty(2 * T * top + 2 * (n_experts + 1), dtype=torch.int32, device=dev)
    ids, order = ints[:T * top], ints[T * top:2 * T * top]
    offsets = ints[2 * T * top:2 * T * top + n_experts + 1]
    tile_off = ints[2 * T * top + n_experts + 1:]
    wts = torch.empty(T * top, dtype=torch.float32, device=dev)
    global _launches
    _launches += 1                      # (two kernels)
    _f32vec(choice_bias, n_experts, "moe_route choice bias")
    _gpu(choice_bias)
    _call("tlc_moe_route", logits.data_ptr(), _rows(logits, "router logits"), T, int(n_experts), int(top), ROUTE_WEIGHTS[weights],
          _p(choice_bias), int(n_identity), ids.data_ptr(),
          wts.data_ptr(), order.data_ptr(), offsets.data_ptr(), tile_off.data_ptr(), int(tile_rows), float(sum_to), _stream())
    return ids, wts, order, offsets, tile_off, int(tile_rows)


def moe_experts(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, routing, top: int, act: torch.Tensor,
                y: torch.Tensor, act_fn: str = "silu", weight_on: str = "input", limit: float = 0.0, alpha: float = 1.0) -> None:
    """y[t, k, :] for every chosen (token, expert) pair: expert_k(weight * x[t]) with weight_on "input", weight *
    expert_k(x[t]) with "output"; w_gate_up [E, 2F, D], w_down [E, D, F]; act [T*top, F] is scratch of the activation
    type, y float32 [T, top, D].  act_fn: "silu" / "gelu_tanh" (act(g) * u), or "swish_clamped": with g = min(g, limit)
    and u held within +-limit, g * sigmoid(alpha * g) * (u + 1)."""
    if act_fn not in MOE_ACTS or weight_on not in ("input", "output"):
        raise KernelError(f"moe_experts: unknown activation '{act_fn}' or weight placement '{weight_on}'")
    code, w_out = MOE_ACTS[act_fn], int(weight_on == "output")
    _gpu(x, w_gate_up, w_down, act, y)
    ids, wts, order, offsets, tile_off, tile_rows = routing
    T, D = x.shape
    E, F2, _ = w_gate_up.shape
    F = F2 if act_fn in UNGATED_ACTS else F2 // 2         # (experts without a gate: w_gate_up is [E, F, D])
    if not w_gate_up.is_contiguous() or not w_down.is_contiguous() or tuple(w_down.shape) != (E, D, F) \
            or w_gate_up.shape[2] != D or w_gate_up.dtype != w_down.dtype:
        raise KernelError("moe_experts: w_gate_up [E, 2F, D] and w_down [E, D, F] contiguous and of one type")
    if not act.is_contiguous() or tuple(act.shape) != (T * top, F) or y.dtype != torch.float32 or not y.is_contiguous() \
            or y.numel() != T * top * D:
        raise KernelError("moe_experts: act [T*top, F] contiguous, y contiguous float32 [T, top, D]")
    ldx = _rows(x, "moe input")
    if _moe_mma_ok(x, w_gate_up, act.dtype, F):
        _call("tlc_moe_experts_mma", x.data_ptr(), ldx, w_gate_up.data_ptr(), w_down.data_ptr(), order.data_ptr(), offsets.data_ptr(),
              tile_off.data_ptr(), wts.data_ptr(), T, E, int(top), F, D, act.data_ptr(), y.data_ptr(), tile_rows, code, w_out,
              float(limit), float(alpha), _stream())
        return
    if tile_rows != 32:
        raise KernelError("moe_experts: the CUDA-core products take a routing made for tiles of 32 rows")
    _call("tlc_moe_gate_up", x.data_ptr(), dtype_code(x.dtype), _rows(x, "moe input"), w_gate_up.data_ptr(),
          dtype_code(w_gate_up.dtype), order.data_ptr(), offsets.data_ptr(), tile_off.data_ptr(), wts.data_ptr(), T, E, int(top),
          F, D, act.data_ptr(), dtype_code(act.dtype), code, w_out, float(limit), float(alpha), _stream())
    _call("tlc_moe_down", act.data_ptr(), dtype_code(act.dtype), w_down.data_ptr(), dtype_code(w_down.dtype), order.data_ptr(),
          offsets.data_ptr(), tile_off.data_ptr(), T, E, int(top), F, D, y.data_ptr(), _stream())


def moe_identity(x: torch.Tensor, routing, top: int, n_experts: int, y: torch.Tensor) -> None:
    """y[t, k, :] = weight * x[t] for every pair that the routing sent to a router output >= n_experts (an expert that
    returns its input); x float32 or the activation type, y float32 [T, top, D]."""
    _gpu(x, y)
    ids, wts = routing[0], routing[1]
    T, D = x.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or y.numel() != T * top * D:
        raise KernelError("moe_identity: y contiguous float32 [T, top, D]")
    _call("tlc_moe_identity", x.data_ptr(), dtype_code(x.dtype), _rows(x, "moe input"), ids.data_ptr(), wts.data_ptr(), T, int(top),
          int(n_experts), D, y.data_ptr(), _stream())


def qk_whole_norm(qkv: torch.Tensor, q_off: int, q_n: int, q_weight: torch.Tensor, k_off: int, k_n: int, k_weight: torch.Tensor,
                  eps: float) -> None:
    """In place on the float32 projection: its q_n query columns from q_off (all heads together) become
    q / sqrt(mean(q^2) + eps) * q_weight, its k_n key columns from k_off likewise."""
    _gpu(qkv, q_weight, k_weight)
    ld = _rows(qkv, "qkv")
    if qkv.dtype != torch.float32 or max(q_off + q_n, k_off + k_n) > max(ld, qkv.shape[1]):
        raise KernelError("qk_whole_norm: a float32 projection that holds the queries and keys")
    _f32vec(q_weight, q_n, "query norm weight")
    _f32vec(k_weight, k_n, "key norm weight")
    _call("tlc_qk_whole_norm", qkv.data_ptr(), ld, int(q_off), int(q_n), q_weight.data_ptr(), int(k_off), int(k_n),
          k_weight.data_ptr(), float(eps), qkv.shape[0], _stream())


# ---- time mixing with a decaying matrix state -------------------------------------------------------------------
MAX_WKV_HEAD_DIM = 256    # wkv.cu: 32 lanes a column x 8 rows a lane


def shift_mix(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor) -> None:
    """out[t, s] = x[t] + (x[t-1] - x[t]) * mu[s]: x float32 [T, D] contiguous, mu float32 [n, D], out [T, n, D]; x[t-1] is
    the row above or, for a sequence's first row of the step, its slot's row of state [n_slots, D] (zeros at position 0),
    which then receives the sequence's last row."""
    _gpu(x, mu, state, out)
    T, D = x.shape
    n = mu.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or state.dtype != torch.float32 or not state.is_contiguous() \
            or state.shape[-1] != D or not out.is_contiguous() or tuple(out.shape) != (T, n, D):
        raise KernelError("shift_mix: x float32 [T, D], state float32 [n_slots, D], out [T, n, D], all contiguous")
    _f32vec(mu, n * D, "shift_mix mu")
    _call("tlc_shift_mix", x.data_ptr(), mu.data_ptr(), n, T, D, step.row_seq.data_ptr(), step.cu_seqlens.data_ptr(),
          step.slots.data_ptr(), step.start_pos.data_ptr(), state.data_ptr(), out.data_ptr(), dtype_code(out.dtype), _stream())


def wkv_scan(rkv: torch.Tensor, r_off: int, k_off: int, v_off: int, decay_log: torch.Tensor, bonus: torch.Tensor,
             state: torch.Tensor, step, H: int, d: int, out: torch.Tensor) -> None:
    """Per (sequence, head): o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(exp(-exp(decay_log_t))) S + k_t v_t^T.
    rkv float32 [T, *] holds r, k, v from their column offsets (H * d each); decay_log float32 [T, H*d]; bonus u float32
    [H, d]; state float32 [n_slots, H, d, d] (zero at position 0; updated in place); out float32 [T, H*d]."""
    _gpu(rkv, decay_log, bonus, state, out)
    T = rkv.shape[0]
    if rkv.dtype != torch.float32 or decay_log.dtype != torch.float32 or out.dtype != torch.float32 \
            or state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (H, d, d):
        raise KernelError("wkv_scan: float32 projections and a contiguous float32 state [n_slots, H, d, d]")
    _f32vec(bonus, H * d, "wkv bonus")
    ld = _rows(rkv, "wkv projections")
    if max(r_off, k_off, v_off) + H * d > max(ld, rkv.shape[1]) or decay_log.shape[1] != H * d:
        raise KernelError("wkv_scan: r, k or v lies outside the projection's row, or the decay has another width")
    _call("tlc_wkv_scan", rkv.data_ptr(), ld, int(r_off), int(k_off), int(v_off), decay_log.data_ptr(), _rows(decay_log, "wkv decay"),
          bonus.data_ptr(), state.data_ptr(), step.cu_seqlens.data_ptr(), step.slots.data_ptr(), step.start_pos.data_ptr(),
          step.n_seqs, int(H), int(d), out.data_ptr(), _out_rows(out, T, H * d, "wkv_scan"), _stream())


# ---- queries, keys and output gate of an attention mixer ---------------------------------------------------
def qk_rotate_norm(qkv: torch.Tensor, q_off: int, k_off: int, H: int, KV: int, stride: int, dim: int, inv_freq: torch.Tensor,
                   interleaved: bool, norm_eps: Optional[float], positions: torch.Tensor, q_weight: Optional[torch.Tensor] = None,
                   k_weight: Optional[torch.Tensor] = None, pre_eps: float = 0.0, amplitude: float = 1.0) -> None:
    """In place on the float32 projection qkv [T, *] (H query heads from column q_off, KV key heads from k_off, heads
    `stride` values apart of which `dim` are in use): turns the pairs of the first 2 * len(inv_freq) dimensions of every
    head by position * inv_freq[i] (neighbours (2i, 2i+1) when interleaved, else (i, i + half)), then, with norm_eps not
    None, divides the head by sqrt(mean(x^2) + norm_eps).  q_weight, k_weight (float32 [dim], both or neither): BEFORE the
    rotation every query head becomes x / sqrt(mean(x^2) + pre_eps) * q_weight and every key head likewise with k_weight.
    amplitude multiplies every cosine and sine."""
    _gpu(qkv, inv_freq, positions, q_weight, k_weight)
    _f32vec(q_weight, dim, "query norm weight")
    _f32vec(k_weight, dim, "key norm weight")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_rotate_norm: the weights of the norm before the rotation come together")
    T = qkv.shape[0]
    _i32(positions, "positions")
    _f32vec(inv_freq, inv_freq.numel(), "rotation inv_freq")
    ld = _rows(qkv, "qkv")
    if qkv.dtype != torch.float32 or max(q_off + H * stride, k_off + KV * stride) > max(ld, qkv.shape[1]):
        raise KernelError("qk_rotate_norm: a float32 projection that holds every head")
    _call("tlc_qk_rotate_norm", qkv.data_ptr(), ld, int(q_off), int(k_off), int(H), int(KV), int(stride), int(dim),
          inv_freq.data_ptr(), 2 * inv_freq.numel(), int(bool(interleaved)), -1.0 if norm_eps is None else float(norm_eps),
          positions.data_ptr(), T, _p(q_weight), _p(k_weight), float(pre_eps), float(amplitude), _stream())


GATES = {"sigmoid": 0, "silu": 1}


def gate_mul(x: torch.Tensor, gate: torch.Tensor, kind: str = "sigmoid") -> None:
    """x[t, c] *= sigmoid(gate[t, c]) (or silu); x [T, n] with dense rows, gate float32 [T, n] (a range of the columns of
    a wider projection will do)."""
    _gpu(x, gate)
    if kind not in GATES:
        raise KernelError(f"gate_mul: unknown gate '{kind}'; known: {sorted(GATES)}")
    T, n = x.shape
    if gate.dtype != torch.float32 or tuple(gate.shape) != (T, n):
        raise KernelError("gate_mul: the gate must be float32 of x's shape")
    _call("tlc_gate_mul", x.data_ptr(), dtype_code(x.dtype), _rows(x, "gate_mul x"), gate.data_ptr(), _rows(gate, "gate"), n, T,
          GATES[kind], _stream())


# ---- gated delta rule ---------------------------------------------------------------------------------------
MAX_DELTA_KEY_DIM = 256   # delta_rule.cu: rows of a head's state that the threads of a column hold in registers


def delta_prepare(qkv: torch.Tensor, q_off: int, k_off: int, G: int, dk: int, l2_eps: float, q_scale: float, proj: torch.Tensor,
                  b_off: int, H: int, beta: torch.Tensor, channel_decay: Optional[torch.Tensor] = None,
                  A: Optional[torch.Tensor] = None) -> None:
    """In place on qkv (float32 [T, *], G query heads of dk values from q_off, G key heads from k_off): every head becomes
    x / sqrt(sum(x^2) + l2_eps), the queries also times q_scale; beta [T, H] float32 = sigmoid(proj[:, b_off : b_off + H]).
    channel_decay float32 [T, H * dk] with A float32 [H]: turned in place into exp(A[h] * softplus(x)), a decay per key
    channel of every head."""
    _gpu(qkv, proj, beta, channel_decay, A)
    if channel_decay is not None:
        if channel_decay.dtype != torch.float32 or tuple(channel_decay.shape) != (qkv.shape[0], H * dk) or A is None:
            raise KernelError("delta_prepare: decays per channel are float32 [T, H * dk] and come with A [H]")
        _f32vec(A, H, "delta_prepare A")
    T = qkv.shape[0]
    if qkv.dtype != torch.float32 or proj.dtype != torch.float32 or beta.dtype != torch.float32 or not beta.is_contiguous() \
            or tuple(beta.shape) != (T, H) or proj.shape[0] != T:
        raise KernelError("delta_prepare: float32 tensors, beta contiguous [T, H]")
    _call("tlc_delta_prepare", qkv.data_ptr(), _rows(qkv, "qkv"), int(q_off), int(k_off), int(G), int(dk), float(l2_eps),
          float(q_scale), proj.data_ptr(), _rows(proj, "proj"), int(b_off), int(H), beta.data_ptr(), T, _p(channel_decay),
          0 if channel_decay is None else _rows(channel_decay, "decays"), _p(A), _stream())


def delta_rule_split(threads: int) -> None:
    """Fixes how many threads of the delta rule's kernel share the rows of a column group of the state (8 or 16; 0:
    chosen: 16 for prompts, 8 for single-token steps); for tests and comparisons."""
    library().tlc_delta_rule_split(int(threads))


def delta_rule(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, beta: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
               step, y: torch.Tensor, H: int, G: int, dk: int, dv: int, per_channel: bool = False) -> None:
    """The gated delta rule over every sequence's rows of the step, from its slot's state [n_slots, H, dk, dv] float32
    (zero at position 0; updated in place): M <- a M; w = b (v - M^T k); M <- M + k w^T; y = M^T q (a the decay, b the
    write strength `beta`; decay [T, H], or [T, H * dk] for a factor per key channel: M <- diag(a) M).  qkv float32
    [T, *] holds the prepared queries and keys (G heads of dk) and the values (H heads of dv); beta, decay float32 [T, H];
    y float32 [T, H*dv]."""
    _gpu(qkv, beta, decay, state, y)
    T = qkv.shape[0]
    if per_channel and (decay.dim() != 2 or decay.shape[1] != H * dk):
        raise KernelError("delta_rule: decays per channel must be float32 [T, H * dk]")
    for t, n in ((beta, "beta"),) + (() if per_channel else ((decay, "decay"),)):
        if t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != (T, H):
            raise KernelError(f"delta_rule: {n} must be contiguous float32 [T, H]")
    if per_channel and (decay.dtype != torch.float32 or decay.shape[0] != T):
        raise KernelError("delta_rule: decays per channel must be float32 [T, H * dk]")
    if qkv.dtype != torch.float32 or state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (H, dk, dv):
        raise KernelError("delta_rule: float32 inputs and a contiguous float32 state [n_slots, H, dk, dv]")
    if y.dtype != torch.float32:
        raise KernelError("delta_rule: y must be float32")
    ldy = _out_rows(y, T, H * dv, "delta_rule")
    _call("tlc_delta_rule", qkv.data_ptr(), _rows(qkv, "qkv"), int(q_off), int(k_off), int(v_off), beta.data_ptr(), decay.data_ptr(),
          state.data_ptr(), step.cu_seqlens.data_ptr(), step.slots.data_ptr(), step.start_pos.data_ptr(), step.n_seqs, T, int(H),
          int(G), int(dk), int(dv), y.data_ptr(), ldy, _rows(decay, "decays") if per_channel else 0, _stream())
