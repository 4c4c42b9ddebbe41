"""ctypes view of the C ABI declared in ``include/rllama_b200.h``.

The shared library is built in-tree by ``rllama_b200.build``. There is no CPU fallback:
importing this module without the built library raises, and every entry point fails with
an ``RllamaError`` when no sm_100 device is usable.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# RLLAMA_B200_LIB selects another build of the same library (the timeline build of ``rllama_b200.build --trace``)
LIB_PATH = os.environ.get("RLLAMA_B200_LIB") or os.path.join(_HERE, "librllama_b200.so")

F32, F16 = 0, 1

# every symbol include/rllama_b200.h declares
EXPORTS = [
    "rlb_last_error", "rlb_device_count",
    "rlb_ctx_create", "rlb_ctx_destroy", "rlb_ctx_flush", "rlb_ctx_kernel_launches",
    "rlb_tensor_upload", "rlb_tensor_zeros", "rlb_tensor_wait", "rlb_tensor_download", "rlb_event_wait", "rlb_tensor_free",
    "rlb_copy_inplace", "rlb_transpose_from", "rlb_hadamard_product_inplace", "rlb_silu_inplace",
    "rlb_matrix_mul_inplace_transposed", "rlb_attention_decode", "rlb_attention_decode_static", "rlb_attention_prefill",
    "rlb_model_create", "rlb_model_set_tensor", "rlb_model_finalize", "rlb_model_free",
    "rlb_tp_nccl_unique_id", "rlb_tp_nccl_init", "rlb_tp_peer_export", "rlb_tp_peer_import", "rlb_tp_peer_import_local", "rlb_tp_set_mode",
    "rlb_caches_create", "rlb_caches_true_clone", "rlb_caches_shift_left", "rlb_caches_free", "rlb_caches_read",
    "rlb_forward", "rlb_forward_greedy", "rlb_decode_greedy",
    "rlb_model_set_option", "rlb_model_get_stat",
    "rlb_data_source_open", "rlb_data_source_free", "rlb_data_source_shards", "rlb_data_source_tensor_shape",
    "rlb_data_source_read_f16", "rlb_model_params_from_json", "rlb_model_from_llama_source",
    "rlb_data_source_open_vicuna", "rlb_data_source_open_inferred", "rlb_data_source_need_antitranspose",
    "rlb_huggingface_antitranspose_f16",
    "rlb_tokenizer_load", "rlb_tokenizer_free", "rlb_tokenizer_n_pieces", "rlb_tokenizer_id_to_str", "rlb_tokenizer_str_to_id",
    "rlb_tokenizer_tokenize_to_ids",
    "rlb_sampler_create", "rlb_sampler_free", "rlb_sampler_set", "rlb_sampler_get", "rlb_sampler_seed", "rlb_sampler_sample",
    "rlb_sampler_candidates",
]


class RllamaError(RuntimeError):
    """A non-zero status from the library (the reference panics or returns Err here)."""

    def __init__(self, status, message):
        super().__init__("rllama_b200 status %d: %s" % (status, message))
        self.status = status


class ModelParams(ctypes.Structure):
    _fields_ = [
        ("dim", ctypes.c_int32), ("n_layers", ctypes.c_int32), ("n_heads", ctypes.c_int32),
        ("ffn_dim", ctypes.c_int32), ("vocab_size", ctypes.c_int32), ("max_seq_len", ctypes.c_int32),
        ("norm_eps", ctypes.c_float), ("force_f16", ctypes.c_int32),
        ("tp_rank", ctypes.c_int32), ("tp_size", ctypes.c_int32),
        ("has_percentage_to_gpu", ctypes.c_int32), ("percentage_to_gpu", ctypes.c_float),
    ]


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "librllama_b200.so is not built (run `python -m rllama_b200.build`); there is no CPU fallback")
    L = ctypes.CDLL(LIB_PATH)
    vp, ci, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int32, ctypes.c_int64
    P = ctypes.POINTER
    L.rlb_last_error.restype = ctypes.c_char_p
    L.rlb_last_error.argtypes = []
    sig = {
        "rlb_device_count": [P(ci)],
        "rlb_ctx_create": [ci, ci, P(vp)], "rlb_ctx_destroy": [vp], "rlb_ctx_flush": [vp],
        "rlb_ctx_kernel_launches": [vp, P(ctypes.c_uint64)],
        "rlb_tensor_upload": [vp, vp, i64, i64, i64, ci, P(vp)],
        "rlb_tensor_zeros": [vp, i64, i64, i64, ci, P(vp)],
        "rlb_tensor_wait": [vp], "rlb_tensor_download": [vp, vp, P(vp)], "rlb_event_wait": [vp], "rlb_tensor_free": [vp],
        "rlb_copy_inplace": [vp, vp], "rlb_transpose_from": [vp, vp], "rlb_hadamard_product_inplace": [vp, vp],
        "rlb_silu_inplace": [vp], "rlb_matrix_mul_inplace_transposed": [vp, vp, vp],
        "rlb_attention_decode": [vp, vp, vp, vp, i32, i32, i32, i32],
        "rlb_attention_decode_static": [vp, vp, vp, vp, i32, i32, i32, i32],
        "rlb_attention_prefill": [vp, vp, vp, vp, i32, i32, i32, i32],
        "rlb_model_create": [vp, P(ModelParams), P(vp)],
        "rlb_model_set_tensor": [vp, ci, i32, vp, i64, i64, i64, ci],
        "rlb_model_finalize": [vp], "rlb_model_free": [vp],
        "rlb_tp_nccl_unique_id": [vp], "rlb_tp_nccl_init": [vp, vp],
        "rlb_tp_peer_export": [vp, vp], "rlb_tp_peer_import": [vp, vp, i32], "rlb_tp_peer_import_local": [vp, vp, i32], "rlb_tp_set_mode": [vp, i32],
        "rlb_caches_create": [vp, P(vp)], "rlb_caches_true_clone": [vp, P(vp)], "rlb_caches_shift_left": [vp, i32],
        "rlb_caches_free": [vp], "rlb_caches_read": [vp, i32, i32, i32, i32, vp],
        "rlb_forward": [vp, vp, vp, i32, i32, vp],
        "rlb_forward_greedy": [vp, vp, vp, i32, i32, P(i32)],
        "rlb_decode_greedy": [vp, vp, i32, i32, i32, vp, P(ctypes.c_float)],
        "rlb_model_set_option": [vp, ctypes.c_char_p, i64],
        "rlb_model_get_stat": [vp, ctypes.c_char_p, P(ctypes.c_double)],
        "rlb_data_source_open": [ctypes.c_char_p, P(vp)], "rlb_data_source_free": [vp],
        "rlb_data_source_shards": [vp, P(i32)],
        "rlb_data_source_tensor_shape": [vp, ctypes.c_char_p, i32, P(i64), P(i64)],
        "rlb_data_source_read_f16": [vp, ctypes.c_char_p, i32, vp, i64, i64],
        "rlb_model_params_from_json": [ctypes.c_char_p, P(ModelParams)],
        "rlb_model_from_llama_source": [vp, vp, P(ModelParams), P(vp)],
        "rlb_data_source_open_vicuna": [ctypes.c_char_p, P(vp)], "rlb_data_source_open_inferred": [ctypes.c_char_p, P(vp)],
        "rlb_data_source_need_antitranspose": [vp, P(i32)],
        "rlb_huggingface_antitranspose_f16": [vp, vp, i64, i64, i32],
        "rlb_tokenizer_load": [ctypes.c_char_p, P(vp)], "rlb_tokenizer_free": [vp], "rlb_tokenizer_n_pieces": [vp, P(i32)],
        "rlb_tokenizer_id_to_str": [vp, i32, P(ctypes.c_char_p)], "rlb_tokenizer_str_to_id": [vp, ctypes.c_char_p, P(i32)],
        "rlb_tokenizer_tokenize_to_ids": [vp, ctypes.c_char_p, vp, i32, P(i32)],
        "rlb_sampler_create": [P(vp)], "rlb_sampler_free": [vp],
        "rlb_sampler_set": [vp, ctypes.c_float, ctypes.c_float, i32, ctypes.c_float],
        "rlb_sampler_get": [vp, P(ctypes.c_float), P(ctypes.c_float), P(i32), P(ctypes.c_float)],
        "rlb_sampler_seed": [vp, ctypes.c_uint64],
        "rlb_sampler_sample": [vp, vp, i32, vp, i32, P(i32), P(ctypes.c_float)],
        "rlb_sampler_candidates": [vp, vp, i32, vp, i32, vp, vp, i32, P(i32)],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.restype = ci
        fn.argtypes = args
    _lib = L
    return L


def check(status):
    if status != 0:
        raise RllamaError(status, lib().rlb_last_error().decode("utf-8", "replace"))
