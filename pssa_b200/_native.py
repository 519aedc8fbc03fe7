"""ctypes binding of include/pssa_b200.h. Fails loudly when the CUDA library is missing: there is
no CPU fallback behind this package."""
import ctypes as C
import pathlib

PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = PKG / "libpssa_b200.so"

OK, ERR_INVALID_ARGUMENT, ERR_SHAPE, ERR_CUDA, ERR_FATAL_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_TOKEN, \
    ERR_CANCELLED, ERR_BANK = range(10)

_fp = C.POINTER(C.c_float)
_vp = C.c_void_p
_sz = C.c_size_t

# name -> (restype, argtypes); every symbol include/pssa_b200.h declares
SIGNATURES = {
    "pssa_b200_ctx_create": (C.c_int32, [C.c_int32, C.POINTER(_vp)]),
    "pssa_b200_ctx_destroy": (None, [_vp]),
    "pssa_b200_last_error": (C.c_char_p, [_vp]),
    "pssa_b200_ctx_set_stream": (C.c_int32, [_vp, _vp]),
    "pssa_b200_ctx_use_own_stream": (C.c_int32, [_vp]),
    "pssa_b200_ctx_synchronize": (C.c_int32, [_vp]),
    "pssa_b200_backend_label": (C.c_char_p, [_vp]),
    "pssa_b200_launch_count": (C.c_uint64, [_vp]),
    "pssa_b200_ctx_reserve": (C.c_int32, [_vp, _sz]),
    "pssa_b200_ctx_set_scan_chunks": (C.c_int32, [_vp, C.c_uint32]),
    "pssa_b200_affine_scan_dev": (C.c_int32, [_vp, _vp, _vp, _sz, _sz, _sz]),
    "pssa_b200_affine_scan": (C.c_int32, [_vp, _vp, _vp, _sz, _sz, _sz]),
    "pssa_b200_scan_states_dev": (C.c_int32, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "pssa_b200_scan_states": (C.c_int32, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "pssa_b200_scan_states_noalloc_dev": (C.c_int32, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, C.c_uint32]),
    "pssa_b200_ssm_forward_dev": (C.c_int32, [_vp] * 11 + [_vp, _vp, _sz, _sz, _sz, _sz, C.c_uint32]),
    "pssa_b200_ssm_forward": (C.c_int32, [_vp] * 7 + [_sz, _sz, _sz] + [_vp] * 4 + [C.c_uint32]),
    "pssa_b200_memory_read_dev": (C.c_int32, [_vp, _vp, C.c_int32, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, C.c_float, _sz,
                                              _vp, _vp, _vp, _vp, _vp, C.c_uint32]),
    "pssa_b200_memory_read_topk_dev": (C.c_int32, [_vp, _vp, C.c_int32, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, C.c_float, _sz,
                                                   _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_uint32]),
    "pssa_b200_memory_read": (C.c_int32, [_vp, _vp, C.c_int32, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, C.c_float, _sz,
                                          _vp, _vp, _vp, _vp, _vp, C.c_uint32]),
    "pssa_b200_memory_forward": (C.c_int32, [_vp] * 10 + [_sz] * 6 + [C.c_float] + [_vp] * 8 + [C.c_int32]),
    "pssa_b200_memory_forward_dev": (C.c_int32, [_vp] * 10 + [_sz] * 6 + [C.c_float] + [_vp] * 8 + [C.c_int32]),
    "pssa_b200_ssm_forward_resident": (C.c_int32, [_vp] * 8 + [_sz, _sz, _sz, C.c_uint32]),
    "pssa_b200_memory_forward_after_ssm": (C.c_int32, [_vp] * 9 + [_sz] * 6 + [C.c_float] + [_vp] * 12 + [C.c_int32]),
    "pssa_b200_bank_insert_protected_dev": (C.c_int32, [_vp] * 7 + [_sz, _sz, _sz] + [_vp] * 4 + [_sz, _vp, _vp, C.c_float]),
    "pssa_b200_adapter_plastic_update_dev": (C.c_int32, [_vp] * 5 + [_sz, _sz]),
    "pssa_b200_adapter_consolidate_dev": (C.c_int32, [_vp, _vp, _vp, _sz, C.c_float]),
    "pssa_b200_ctx_poll_status": (C.c_int32, [_vp]),
    "pssa_b200_ctx_selftest_wait_expiry": (C.c_int32, [_vp, C.c_uint32]),
    "pssa_b200_gemm_xwt": (C.c_int32, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, C.c_int32, C.c_float, C.c_int32]),
    "pssa_b200_gemm_xwt_dev": (C.c_int32, [_vp, _vp, _vp, _sz, _sz, _sz, _vp, _sz, C.c_int32, C.c_float, C.c_int32]),
    "pssa_b200_model_create": (C.c_int32, [_vp, _vp, C.c_uint32, C.POINTER(_vp)]),
    "pssa_b200_model_destroy": (None, [_vp]),
    "pssa_b200_model_set_tensor": (C.c_int32, [_vp, C.c_int32, C.c_int32, _vp, _sz]),
    "pssa_b200_model_insert_memory": (C.c_int32, [_vp, C.c_uint32, C.c_float, C.c_uint64, _vp]),
    "pssa_b200_model_sampler_push": (C.c_int32, [_vp, C.c_uint32, _vp, _sz]),
    "pssa_b200_model_reserve": (C.c_int32, [_vp, _sz, _sz]),
    "pssa_b200_model_get_tensor": (C.c_int32, [_vp, C.c_int32, C.c_int32, _vp, _sz]),
    "pssa_b200_model_init_random": (C.c_int32, [_vp, C.c_uint64, C.POINTER(C.c_uint64)]),
    "pssa_b200_model_set_bank": (C.c_int32, [_vp, C.c_int32, _vp, _vp, _vp, C.c_uint64, C.c_uint64, _vp, _vp]),
    "pssa_b200_model_set_top_k": (C.c_int32, [_vp, _sz]),
    "pssa_b200_model_set_precision": (C.c_int32, [_vp, C.c_int32]),
    "pssa_b200_model_set_option": (C.c_int32, [_vp, C.c_int32, C.c_int32]),
    "pssa_b200_model_set_max_rows": (C.c_int32, [_vp, _sz]),
    "pssa_b200_model_reset_state": (C.c_int32, [_vp, C.c_uint32]),
    "pssa_b200_model_get_state": (C.c_int32, [_vp, C.c_uint32, _vp, _sz]),
    "pssa_b200_model_set_state": (C.c_int32, [_vp, C.c_uint32, _vp, _sz]),
    "pssa_b200_model_prefill": (C.c_int32, [_vp, C.c_uint32, _vp, _sz, _vp, C.POINTER(_sz), _vp, _vp]),
    "pssa_b200_model_prefill_batch": (C.c_int32, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "pssa_b200_model_prefill_batch_dev": (C.c_int32, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "pssa_b200_ctx_profile_begin": (C.c_int32, [_vp]),
    "pssa_b200_ctx_profile_end": (C.c_int32, [_vp, C.POINTER(C.c_uint32)]),
    "pssa_b200_ctx_profile_row": (C.c_int32, [_vp, C.c_uint32, C.POINTER(C.c_char_p), C.POINTER(C.c_uint64),
                                              C.POINTER(C.c_double)]),
    "pssa_b200_model_decode_step": (C.c_int32, [_vp, _vp, _vp, _sz, _vp, _vp]),
    "pssa_b200_sample_dev": (C.c_int32, [_vp, _vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_uint32]),
    "pssa_b200_model_score": (C.c_int32, [_vp, C.c_uint32, _vp, _vp, _sz, _vp, _vp, _vp]),
    "pssa_b200_model_set_observer": (C.c_int32, [_vp, C.c_int32]),
    "pssa_b200_model_get_observation": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, _vp, _vp, _vp, _vp]),
    "pssa_b200_model_sampler_seed": (C.c_int32, [_vp, C.c_uint32, C.c_uint64]),
    "pssa_b200_model_decode_step_sampled": (C.c_int32, [_vp, _vp, _vp, _sz, _vp, C.c_uint32, _vp, _vp]),
    "pssa_b200_checkpoint_probe": (C.c_int32, [_vp, _sz, _vp, _vp, _vp, _sz]),
    "pssa_b200_model_load_checkpoint": (C.c_int32, [_vp, _vp, _sz, C.c_uint32, _vp]),
    "pssa_b200_model_set_seqpar": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, _vp, _vp, _sz, _vp, _vp]),
}
SSM_EXACT = 1
MEM_EXACT = 1
MEM_F32_DISTANCE = 2
MEM_TC_DISTANCE = 4
MEM_NO_FUSED = 8
MEM_HANDOVER_SELFTEST = 16
MEM_PHASE_CLOCKS = 32
EPI_NONE, EPI_SOFTPLUS, EPI_SIGMOID, EPI_SILU, EPI_SCALE, EPI_ADD_OUT = range(6)
PRECISION_BF16, PRECISION_FP32_EXACT = 0, 1
CANCEL_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p)
EXCHANGE_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)


class Sampling(C.Structure):
    """`pssa_b200_sampling`"""
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_uint32), ("repetition_penalty", C.c_float)]


SAMPLE_EXACT = 1


class Config(C.Structure):
    """`pssa_b200_config`"""
    _fields_ = [("depth", C.c_uint64), ("d_vocab", C.c_uint64), ("d_latent", C.c_uint64), ("d_state", C.c_uint64),
                ("d_mem_key", C.c_uint64), ("mem_capacity", C.c_uint64), ("tau_mem", C.c_float), ("reserved", C.c_uint32)]

_lib = None


def lib() -> C.CDLL:
    """Load libpssa_b200.so (built in-tree by pssa_b200.build). Raises if it is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m pssa_b200.build` (needs nvcc). "
                "The B200 path has no CPU fallback.")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class B200Error(RuntimeError):
    """A non-zero status from the C ABI; `.status` holds the code, the text is the library's message."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
