"""ctypes binding of ``libcgpt_b200.so`` (the C ABI declared in ``include/cgpt_b200.h``).

There is no fallback: if the shared library is missing the import fails with the build command to
run, and every op raises if the library reports an error.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch  # noqa: F401  (loads libcudart.so.12 first so the library binds to the same runtime)

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libcgpt_b200.so"

F16, BF16, F32 = 0, 1, 2
_TORCH_TO_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}

ERRORS = {
    1: "null pointer", 2: "unsupported dtype", 3: "invalid shape", 4: "invalid option",
    5: "misaligned pointer", 6: "unsupported configuration", 7: "invalid state",
    8: "device-side wait timed out",
}


class CgptError(RuntimeError):
    """A CUDA runtime/driver failure reported by the library (negative status)."""


class CgptInvalidArgument(ValueError):
    """An argument error class reported by the library (positive status); the reference throws
    std::invalid_argument for the same conditions."""


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m cgpt_b200.build` (needs nvcc; no GPU required). "
            "cgpt_b200 has no CPU or PyTorch fallback."
        )
    return C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)


lib = _load()

_vp, _sz, _i, _f, _u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_uint64


class AdamWTensor(C.Structure):
    _fields_ = [("param", _vp), ("grad", _vp), ("master", _vp), ("m", _vp), ("v", _vp),
                ("count", C.c_uint64), ("dtype", C.c_int32), ("reserved", C.c_int32)]


class AdamWOptions(C.Structure):
    _fields_ = [("learning_rate", _f), ("beta1", _f), ("beta2", _f), ("epsilon", _f),
                ("weight_decay", _f), ("loss_scale", _f), ("max_grad_norm", _f)]


BLOCK_PARAM_FIELDS = ("attention_norm", "q_projection", "k_projection", "q_norm", "k_norm", "v_projection",
                      "o_projection", "ffn_norm", "gate_proj", "up_proj", "down_proj")
BLOCK_SAVED_FIELDS = ("norm", "query", "key", "value", "query_pre_norm", "key_pre_norm", "attention_output",
                      "attention_logsumexp", "gate", "up", "activated", "attention_norm_output")


class BlockParams(C.Structure):
    _fields_ = [(n, _vp) for n in BLOCK_PARAM_FIELDS]


class BlockSaved(C.Structure):
    _fields_ = [(n, _vp) for n in BLOCK_SAVED_FIELDS]


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("vocab", "layers", "hidden", "intermediate", "q_heads", "kv_heads",
                                          "head_dim", "rotary_dim", "max_seq")] + \
               [("rms_epsilon", _f), ("dtype", C.c_int32), ("tied_embeddings", C.c_int32), ("reserved", C.c_int32)]


class ModelTensors(C.Structure):
    _fields_ = [("token_embedding", _vp), ("layers", C.POINTER(BlockParams)), ("final_norm", _vp), ("lm_head", _vp)]


class ModelSaved(C.Structure):
    _fields_ = [("layers", C.POINTER(BlockSaved)), ("layer_inputs", C.POINTER(_vp)), ("hidden", _vp),
                ("normalized", _vp)]


_pBP, _pBS, _pMC, _pMT, _pMS = (C.POINTER(BlockParams), C.POINTER(BlockSaved), C.POINTER(ModelConfig),
                                C.POINTER(ModelTensors), C.POINTER(ModelSaved))

SIGNATURES = {
    "cgpt_cut_cross_entropy": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _f, _i, _sz, _i, _vp]),
    "cgpt_cut_cross_entropy_form": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _f, _i, _sz, _i, _vp]),
    "cgpt_block_workspace_bytes": (_sz, [_pMC, _sz, _sz]),
    "cgpt_block_forward": (_i, [_vp, _vp, _pBP, _pBS, _vp, _vp, _vp, _pMC, _sz, _sz, _sz, _vp]),
    "cgpt_block_backward": (_i, [_vp, _vp, _vp, _pBP, _pBP, _pBS, _vp, _vp, _vp, _pMC, _sz, _sz, _sz, _vp]),
    "cgpt_model_forward": (_i, [_vp, _vp, _pMT, _pMS, _vp, _vp, _vp, _pMC, _sz, _sz, _vp]),
    "cgpt_model_backward": (_i, [_vp, _vp, _vp, _pMT, _pMT, _pMS, _vp, _vp, _vp, _pMC, _sz, _sz, _vp]),
    "cgpt_model_backward_steps": (_i, [_vp, _vp, _vp, _pMT, _pMT, _pMS, _vp, _vp, _vp, _pMC, _sz, _sz, _sz, _sz, _vp]),
    "cgpt_b200_version": (C.c_char_p, []),
    "cgpt_b200_launch_count": (C.c_uint64, []),
    "cgpt_b200_device_status": (_i, [C.POINTER(C.c_uint), _i]),
    "cgpt_b200_reserve_scratch": (_i, [_sz]),
    "cgpt_b200_set_branch_streams": (_i, [_i]),
    "cgpt_b200_gemm_timing": (_i, [_i]),
    "cgpt_b200_gemm_timing_read": (_i, [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(_u64)]),
    "cgpt_gemm": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _i, _vp]),
    "cgpt_linear_forward": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _i, _vp]),
    "cgpt_linear_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _vp]),
    "cgpt_linear_forward_fused": (_i, [C.POINTER(_vp), _vp, C.POINTER(_vp), C.POINTER(_sz), _sz, _sz, _sz, _i, _vp]),
    "cgpt_linear_backward_weight_fused": (_i, [C.POINTER(_vp), C.POINTER(_vp), _vp, C.POINTER(_sz), _sz, _sz, _sz, _i, _i, _vp]),
    "cgpt_linear_swiglu_forward": (_i, [_vp] * 6 + [_sz] * 3 + [_i, _vp]),
    "cgpt_linear_backward_input_fused": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_sz), _sz, _sz, _sz, _i, _i, _vp]),
    "cgpt_linear_forward_sum": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_sz), _sz, _sz, _sz, _vp, _i, _vp]),
    "cgpt_attention_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _f, _i, _sz, _i, _i, _vp]),
    "cgpt_attention_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _f, _i,
                                     _sz, _i, _i, _i, _vp]),
    "cgpt_rmsnorm_forward": (_i, [_vp, _vp, _vp, _sz, _sz, _f, _i, _vp]),
    "cgpt_rmsnorm_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _vp]),
    "cgpt_rmsnorm_backward_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _vp]),
    "cgpt_rmsnorm_forward_dual": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _vp]),
    "cgpt_rmsnorm_backward_dual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _vp]),
    "cgpt_qknorm_rope_forward": (_i, [_vp] * 8 + [_sz] * 8 + [_f, _i, _vp]),
    "cgpt_qknorm_rope_backward": (_i, [_vp] * 12 + [_sz] * 8 + [_f, _i, _vp]),
    "cgpt_rope_forward": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _i, _vp]),
    "cgpt_rope_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _i, _vp]),
    "cgpt_swiglu_forward": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "cgpt_swiglu_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _vp]),
    "cgpt_embedding_forward": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _i, _vp]),
    "cgpt_embedding_backward": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _i, _i, _i, _vp]),
    "cgpt_add": (_i, [_vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "cgpt_cross_entropy": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _vp]),
    "cgpt_adamw_create": (_i, [C.POINTER(_vp), C.POINTER(AdamWTensor), _sz, _u64, _vp]),
    "cgpt_adamw_destroy": (_i, [_vp]),
    "cgpt_adamw_step": (_i, [_vp, C.POINTER(AdamWOptions), _vp]),
    "cgpt_adamw_step_device_lr": (_i, [_vp, C.POINTER(AdamWOptions), _vp, _vp]),
    "cgpt_adamw_check": (_i, [_vp, C.POINTER(_u64), C.POINTER(_i), _vp]),
    "cgpt_adamw_last_stats": (_i, [_vp, C.POINTER(_f), C.POINTER(_f), _vp]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def check(status: int, what: str) -> None:
    """Raises for a non-zero status of a library call."""
    if status == 0:
        return
    if status > 0:
        raise CgptInvalidArgument(f"{what}: {ERRORS.get(status, 'error ' + str(status))}")
    raise CgptError(f"{what}: CUDA error {-status}")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _TORCH_TO_CODE[t.dtype]
    except KeyError:
        raise CgptInvalidArgument(f"unsupported dtype {t.dtype}") from None


def ptr(t) -> int | None:
    """Device pointer of a tensor (None passes NULL)."""
    if t is None:
        return None
    if not t.is_contiguous():
        raise CgptInvalidArgument("tensor must be contiguous")
    return t.data_ptr()


def stream_ptr(stream=None) -> int:
    """cudaStream_t of `stream` (a torch.cuda.Stream) or of torch's current stream."""
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream


def device_status(clear: bool = True) -> int:
    """Status word of the tensor-core kernels: non-zero if a bounded device-side wait ran out."""
    v = C.c_uint(0)
    check(lib.cgpt_b200_device_status(C.byref(v), int(clear)), "device_status")
    return int(v.value)


def launch_count() -> int:
    return int(lib.cgpt_b200_launch_count())
