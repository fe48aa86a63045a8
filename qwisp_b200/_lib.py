"""ctypes binding of libseedless_b200.so (declarations follow include/seedless_b200.h)."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libseedless_b200.so")

SL_OK, SL_ERR_INVALID, SL_ERR_NO_DEVICE, SL_ERR_CUDA, SL_ERR_POISONED, SL_ERR_CAPACITY, SL_ERR_NOT_FOUND, SL_ERR_FORMAT = 0, -1, -2, -3, -4, -5, -6, -7
_ERR_NAMES = {-1: "invalid argument", -2: "no CUDA device", -3: "CUDA failure", -4: "engine poisoned",
              -5: "capacity exceeded", -6: "unknown tensor", -7: "malformed state blob"}


class SeedlessError(RuntimeError):
    def __init__(self, code, where, fault=None):
        self.code = code
        msg = f"{where}: {_ERR_NAMES.get(code, 'error')} ({code})"
        if fault:
            msg += f" -- {fault}"
        super().__init__(msg)


SL_FLAG_NO_GRAPH, SL_FLAG_NO_PDL, SL_FLAG_STEP_KERNEL, SL_FLAG_SPLIT_EXPERTS, SL_FLAG_ROUTE_IN_ROUTER, SL_FLAG_L2_PREFETCH = 1, 2, 4, 8, 16, 32
SL_FLAG_PASS_KERNELS = 64


class SlConfig(C.Structure):
    _fields_ = [
        ("hidden", C.c_int32), ("n_layers", C.c_int32), ("attn_every", C.c_int32), ("vocab", C.c_int32),
        ("n_experts", C.c_int32), ("top_k", C.c_int32), ("moe_inter", C.c_int32),
        ("gdn_k_heads", C.c_int32), ("gdn_v_heads", C.c_int32),
        ("attn_heads", C.c_int32), ("attn_kv_heads", C.c_int32),
        ("rope_theta", C.c_float), ("rms_eps", C.c_float),
        ("max_rows", C.c_int32), ("max_streams", C.c_int32), ("kv_page_size", C.c_int32), ("kv_pages", C.c_int32),
        ("flags", C.c_int32),
    ]


class SlWeightDesc(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("nbytes", C.c_uint64), ("on_device", C.c_int32)]


class SlSynthSpec(C.Structure):
    _fields_ = [("seed", C.c_uint64), ("norm_jitter", C.c_float), ("conv_std", C.c_float)]


class SlSnap(C.Structure):
    _fields_ = [("kv_len", C.c_int32), ("parity", C.c_int32), ("valid", C.c_int32), ("calls", C.c_int32)]


# every symbol include/seedless_b200.h declares: name -> (restype, argtypes)
_VP, _I32, _I64, _U64, _F = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float
SYMBOLS = {
    "sl_engine_create": (_I32, [C.POINTER(SlConfig), C.POINTER(SlWeightDesc), _I32, C.POINTER(_VP)]),
    "sl_engine_create_synthetic": (_I32, [C.POINTER(SlConfig), C.POINTER(SlSynthSpec), C.POINTER(_VP)]),
    "sl_engine_destroy": (_I32, [_VP]),
    "sl_engine_set_cuda_stream": (_I32, [_VP, _VP]),
    "sl_engine_read_tensor": (_I32, [_VP, C.c_char_p, _VP, _U64]),
    "sl_engine_tensor_bytes": (_I32, [_VP, C.c_char_p, C.POINTER(_U64)]),
    "sl_last_fault": (C.c_char_p, [_VP]),
    "sl_inject_fault": (_I32, [_VP, _I32]),
    "sl_engine_launch_count": (_I64, [_VP]),
    "sl_engine_use_graphs": (_I32, [_VP, _I32]),
    "sl_profile_start": (_I32, [_VP]),
    "sl_profile_report": (_I32, [_VP, C.c_char_p, _U64]),
    "sl_stream_create": (_I32, [_VP, _I32, C.POINTER(_VP)]),
    "sl_stream_destroy": (_I32, [_VP]),
    "sl_stream_len": (_I32, [_VP]),
    "sl_stream_reset": (_I32, [_VP]),
    "sl_forward": (_I32, [_VP, _VP, _I32, _VP]),
    "sl_forward_hybrid": (_I32, [_VP, _VP, _I32, _VP]),
    "sl_hybrid_chunk": (_I32, [_VP]),
    "sl_debug_wait_timeout": (_I32, [_VP]),
    "sl_engine_use_persistent": (_I32, [_VP, _I32]),
    "sl_debug_step_timeline": (_I32, [_VP, _I32, _VP, _U64]),
    "sl_step_argmax": (_I32, [_VP, _VP, _I32, _VP]),
    "sl_chained_step_argmax": (_I32, [_VP, _I32, _I32, _VP]),
    "sl_chained_enqueue": (_I32, [_VP, _I32, _I32]),
    "sl_chained_collect": (_I32, [_VP, _I32, _VP]),
    "sl_step_logits": (_I32, [_VP, _VP, _I32, _VP]),
    "sl_snapshot": (_I32, [_VP, C.POINTER(SlSnap)]),
    "sl_rollback_one_step": (_I32, [_VP, C.POINTER(SlSnap)]),
    "sl_full_snapshot": (_I32, [_VP, C.POINTER(_VP)]),
    "sl_full_restore": (_I32, [_VP, _VP]),
    "sl_fullsnap_free": (_I32, [_VP]),
    "sl_state_size": (_I32, [_VP, C.POINTER(_U64)]),
    "sl_state_save": (_I32, [_VP, _VP, _U64]),
    "sl_state_restore": (_I32, [_VP, _VP, _U64]),
    "sl_batch_step_argmax": (_I32, [_VP, C.POINTER(_VP), _VP, _I32, _VP]),
    "sl_op_qmm4": (_I32, [_VP, _VP, _VP, _VP, _I32, _I32, _I32, _VP]),
    "sl_step_sample_rows": (_I32, [_VP, _VP, _I32, _VP, _VP, _F, _F, C.c_uint32, C.c_uint32, C.c_uint32, _VP, _VP, _VP]),
    "sl_op_sample_rows": (_I32, [_VP, _VP, _I32, _VP, _VP, _F, _F, C.c_uint32, C.c_uint32, C.c_uint32, _VP, _VP, _VP]),
    "sl_ep_unique_id": (_I32, [_VP]),
    "sl_ep_init": (_I32, [_VP, _I32, _I32, _VP, _I32]),
    "sl_op_qmm4_device": (_I32, [_VP, _VP, _VP, _I32, _I32, _I32, _VP, _VP]),
    "sl_op_qmm4_tc_device": (_I32, [_VP, _VP, _VP, _I32, _I32, _I32, _VP, _VP]),
    "sl_op_repack_q4_device": (_I32, [_VP, _VP, _VP, _I32, _I32, _VP, _VP, _VP]),
    "sl_op_quantize_q4": (_I32, [_VP, _I64, _I64, _VP, _VP, _VP]),
    "sl_op_moe_block": (_I32, [_VP, _I32, _VP, _I32, _VP, _VP, _VP]),
    "sl_op_mixer": (_I32, [_VP, _I32, _VP, _I32, _I32, _VP]),
    "sl_op_lm_head": (_I32, [_VP, _VP, _I32, _VP, _VP]),
    "sl_op_lm_head_argmax_static": (_I32, [_VP, _VP, _VP, _I32, _I32, _I32, _VP, _VP]),
    "sl_op_read_kv": (_I32, [_VP, _I32, _I32, _I32, _VP, _VP]),
    "sl_op_layer": (_I32, [_VP, _I32, _VP, _I32, _I32, _VP]),
    "sl_op_head": (_I32, [_VP, _VP, _I32, _VP, _VP]),
    "sl_synth_tokens": (_I32, [_U64, C.c_char_p, _I64, _I32, _VP]),
    "sl_synth_f16": (_I32, [_U64, C.c_char_p, _I64, _F, _F, _VP]),
}

_lib = None


def lib():
    """Load the CUDA library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -m qwisp_b200.build` (nvcc, sm_100a). "
                "qwisp_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)       # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def config(hidden=2048, n_layers=40, attn_every=4, vocab=151936, n_experts=256, top_k=8, moe_inter=512,
           gdn_k_heads=16, gdn_v_heads=32, attn_heads=16, attn_kv_heads=2, rope_theta=1e7, rms_eps=1e-6,
           max_rows=64, max_streams=4, kv_page_size=64, kv_pages=256, flags=0):
    """Geometry of the synthetic 35B-A3B-shaped model by default."""
    return SlConfig(hidden, n_layers, attn_every, vocab, n_experts, top_k, moe_inter, gdn_k_heads, gdn_v_heads,
                    attn_heads, attn_kv_heads, rope_theta, rms_eps, max_rows, max_streams, kv_page_size, kv_pages, flags)


def synth_spec(seed=0, norm_jitter=0.0, conv_std=0.02):
    return SlSynthSpec(seed, norm_jitter, conv_std)
