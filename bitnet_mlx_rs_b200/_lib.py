"""ctypes binding of libbitnet_cuda_kernels.so (the C ABI in include/bitnet_cuda.h).

The library is the product: there is no Python or CPU fallback.  Loading fails loudly
when the shared object has not been built (``python -m bitnet_mlx_rs_b200.build``).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libbitnet_cuda_kernels.so"

sz, i32, u32, f32, vp = C.c_size_t, C.c_int32, C.c_uint32, C.c_float, C.c_void_p

# status codes (include/bitnet_cuda.h)
OK = 0
ERR_CUDA_NOT_ENABLED, ERR_CUDA_DRIVER, ERR_DEVICE, ERR_MEMORY_ALLOCATION, ERR_KERNEL_EXECUTION = 1, 2, 3, 4, 5
ERR_INVALID_CONFIG, ERR_UNSUPPORTED_OPERATION, ERR_STREAM_SYNC, ERR_UNSUPPORTED_DTYPE = 6, 7, 8, 9
ERR_INCOMPATIBLE_SHAPES, ERR_PERFORMANCE, ERR_NULL_POINTER, ERR_WORKSPACE = 10, 11, 12, 13

PATH_AUTO, PATH_DECODE, PATH_PREFILL, PATH_GENERIC, PATH_CLUSTER = 0, 1, 2, 3, 4
FLAG_PDL = 1
FLAG_THROUGHPUT = 2


class ForwardOpts(C.Structure):
    _fields_ = [("path", i32), ("flags", u32), ("q_out_dev", vp), ("a_scale_out_dev", vp),
                ("acc_out_dev", vp), ("ldy", sz), ("stages", i32), ("n_peers", i32), ("y_peers_dev", vp * 8)]


class DeviceInfo(C.Structure):
    _fields_ = [("device_id", i32), ("cc_major", i32), ("cc_minor", i32), ("sm_count", i32),
                ("l2_bytes", i32), ("max_smem_per_block", i32), ("free_bytes", sz), ("total_bytes", sz),
                ("name", C.c_char * 128)]


class W2A8Config(C.Structure):
    _fields_ = [("block_size", u32), ("grid_strategy", i32), ("grid_fixed", u32),
                ("enable_weight_permutation", i32), ("enable_dp4a", i32), ("coalescing_level", i32)]


class BackendConfig(C.Structure):
    _fields_ = [("device_id", sz), ("memory_pool_size", sz), ("num_streams", sz),
                ("enable_profiling", i32), ("w2a8_config", W2A8Config)]


class PerformanceStats(C.Structure):
    _fields_ = [("total_w2a8_operations", C.c_uint64), ("average_execution_time_us", f32),
                ("memory_utilization_percent", f32), ("peak_bandwidth_gbps", f32)]


class RowGlue(C.Structure):
    _fields_ = [("residual_dev", vp), ("sum_out_dev", vp), ("norm_weight_dev", vp), ("norm_bias_dev", vp),
                ("norm_eps", f32), ("normed_out_dev", vp)]


class Stack(C.Structure):
    _fields_ = [("n_members", i32), ("rows", sz * 3), ("scales", f32 * 3)]


class SamplingConfig(C.Structure):
    _fields_ = [("temperature", f32), ("top_k", u32), ("top_p", f32), ("seed", C.c_uint64), ("deterministic", i32)]


class DecoderConfig(C.Structure):
    _fields_ = [("vocab_size", sz), ("hidden_size", sz), ("num_layers", sz), ("num_heads", sz), ("num_kv_heads", sz),
                ("head_dim", sz), ("ffn_size", sz), ("max_seq_len", sz), ("max_batch", sz), ("norm_eps", f32)]


class DecoderLayer(C.Structure):
    _fields_ = [("q_packed", vp), ("k_packed", vp), ("v_packed", vp), ("o_packed", vp),
                ("gate_packed", vp), ("up_packed", vp), ("down_packed", vp),
                ("q_scale", f32), ("k_scale", f32), ("v_scale", f32), ("o_scale", f32),
                ("gate_scale", f32), ("up_scale", f32), ("down_scale", f32),
                ("input_norm_weight", vp), ("input_norm_bias", vp), ("post_norm_weight", vp), ("post_norm_bias", vp)]


DECODER_LOGITS, DECODER_HIDDEN, DECODER_POSITIONS, DECODER_KEY_CACHE, DECODER_VALUE_CACHE = 0, 1, 2, 3, 4


class FfnCall(C.Structure):
    _fields_ = [("gate", vp), ("up", vp), ("down", vp), ("M", sz), ("x_host", vp), ("y_host", vp)]


class BitLinearGroupMember(C.Structure):
    _fields_ = [("packed_dev", vp), ("w_scale", f32), ("x_dev", vp), ("y_dev", vp), ("M", sz), ("ldy", sz)]


class FfnGroupMember(C.Structure):
    _fields_ = [("gate_packed_dev", vp), ("up_packed_dev", vp), ("down_packed_dev", vp), ("gate_scale", f32), ("up_scale", f32),
                ("down_scale", f32), ("x_dev", vp), ("y_dev", vp), ("M", sz)]


_P = C.POINTER
SIGNATURES = {
    "bitnet_is_recoverable": (i32, [i32]),
    "bitnet_status_string": (C.c_char_p, [i32]),
    "bitnet_last_error_string": (C.c_char_p, []),
    "bitnet_device_count": (i32, [_P(i32)]),
    "bitnet_query_device": (i32, [i32, _P(DeviceInfo)]),
    "bitnet_device_error_flags": (i32, [_P(u32)]),
    "bitnet_w2a8_gemv": (i32, [vp, vp, vp, sz, sz, vp]),
    "launch_w2a8_gemv_optimized": (None, [vp, vp, vp, sz, sz, vp]),
    "bitnet_bitlinear_forward": (i32, [vp, f32, vp, vp, sz, sz, sz, _P(ForwardOpts), vp, sz, vp]),
    "bitnet_bitlinear_workspace_size": (i32, [sz, sz, sz, i32, _P(sz)]),
    "bitnet_bitlinear_forward_static": (i32, [vp, f32, vp, vp, sz, sz, sz, vp]),
    "bitnet_quantize_activations": (i32, [vp, sz, sz, vp, vp, vp]),
    "bitnet_ffn_forward": (i32, [vp, f32, vp, f32, vp, f32, vp, vp, vp, sz, sz, sz, _P(ForwardOpts), vp, sz, vp]),
    "bitnet_ffn_workspace_size": (i32, [sz, sz, sz, i32, _P(sz)]),
    "bitnet_pack_ternary": (i32, [vp, sz, vp, vp]),
    "bitnet_unpack_ternary": (i32, [vp, sz, vp, vp]),
    "bitnet_sanitize_packed": (i32, [vp, sz, vp, vp]),
    "bitnet_prepare_weights": (i32, [vp, sz, sz, i32, vp, vp, vp]),
    "bitnet_backend_config_default": (None, [_P(BackendConfig)]),
    "bitnet_backend_create": (i32, [_P(BackendConfig), _P(vp)]),
    "bitnet_backend_destroy": (None, [vp]),
    "bitnet_backend_stream": (i32, [vp, sz, _P(vp)]),
    "bitnet_backend_synchronize": (i32, [vp]),
    "bitnet_backend_get_performance_stats": (i32, [vp, _P(PerformanceStats)]),
    "bitnet_backend_allocate": (i32, [vp, sz, _P(vp)]),
    "bitnet_backend_free": (i32, [vp, vp]),
    "bitnet_backend_copy_to_device": (i32, [vp, vp, vp, sz]),
    "bitnet_backend_copy_to_host": (i32, [vp, vp, vp, sz]),
    "bitnet_backend_memory_usage": (i32, [vp, _P(sz), _P(sz)]),
    "bitnet_backend_w2a8_gemv": (i32, [vp, vp, sz, vp, sz, vp, sz, sz, sz, sz]),
    "bitnet_backend_upload_packed": (i32, [vp, vp, sz, sz, f32, _P(vp)]),
    "bitnet_backend_upload_ternary": (i32, [vp, vp, sz, sz, f32, _P(vp)]),
    "bitnet_backend_upload_f32": (i32, [vp, vp, sz, sz, _P(vp)]),
    "bitnet_backend_upload_gguf_ternary": (i32, [vp, vp, sz, sz, sz, _P(f32), _P(vp)]),
    "bitnet_quantize_pack_weights": (i32, [vp, sz, vp, vp, vp, sz, vp]),
    "bitnet_quantize_pack_weights_workspace_size": (i32, [sz, _P(sz)]),
    "bitnet_backend_free_weights": (i32, [vp, vp]),
    "bitnet_weights_info": (i32, [vp, _P(sz), _P(sz), _P(f32), _P(vp)]),
    "bitnet_backend_bitlinear_forward": (i32, [vp, vp, vp, vp, sz, _P(ForwardOpts), sz]),
    "bitnet_backend_bitlinear_forward_host": (i32, [vp, vp, vp, vp, sz, _P(ForwardOpts), sz]),
    "bitnet_backend_ffn_forward_host": (i32, [vp, vp, vp, vp, vp, vp, sz, _P(ForwardOpts), sz]),
    "bitnet_backend_ffn_forward_host_async": (i32, [vp, vp, vp, vp, vp, vp, sz, _P(ForwardOpts), sz]),
    "bitnet_bitlinear_forward_fused": (i32, [vp, _P(Stack), vp, _P(RowGlue), vp, sz, sz, _P(ForwardOpts), vp, sz, vp]),
    "bitnet_bitlinear_fused_workspace_size": (i32, [sz, sz, sz, i32, _P(sz)]),
    "bitnet_ffn_forward_fused": (i32, [vp, f32, vp, f32, vp, f32, vp, _P(RowGlue), vp, vp, sz, sz, sz, _P(ForwardOpts), vp, sz, vp]),
    "bitnet_ffn_fused_workspace_size": (i32, [sz, sz, sz, i32, _P(sz)]),
    "bitnet_row_glue_forward": (i32, [vp, sz, sz, _P(RowGlue), vp]),
    "bitnet_attention_decode": (i32, [vp, sz, sz, sz, vp, vp, vp, vp, sz, sz, sz, sz, sz, i32, vp, sz, vp]),
    "bitnet_attention_scratch_size": (i32, [sz, sz, sz, sz, i32, _P(sz)]),
    "bitnet_attention_splits": (i32, [sz, sz, sz]),
    "bitnet_sampling_config_default": (None, [_P(SamplingConfig)]),
    "bitnet_sample_tokens": (i32, [vp, sz, sz, _P(SamplingConfig), vp, vp, vp]),
    "bitnet_seed_sampler": (i32, [vp, sz, C.c_uint64, vp]),
    "bitnet_decoder_config_default": (None, [_P(DecoderConfig)]),
    "bitnet_decoder_create": (i32, [vp, _P(DecoderConfig), _P(vp)]),
    "bitnet_decoder_destroy": (None, [vp]),
    "bitnet_decoder_load_embedding": (i32, [vp, vp]),
    "bitnet_decoder_load_layer": (i32, [vp, sz, _P(DecoderLayer)]),
    "bitnet_decoder_load_lm_head": (i32, [vp, vp, f32]),
    "bitnet_decoder_reset": (i32, [vp]),
    "bitnet_decoder_set_graphs": (i32, [vp, i32]),
    "bitnet_decoder_feed": (i32, [vp, vp, sz, sz]),
    "bitnet_decoder_decode": (i32, [vp, vp, sz, sz, _P(SamplingConfig), i32, vp, _P(sz)]),
    "bitnet_decoder_generate": (i32, [vp, vp, sz, sz, sz, _P(SamplingConfig), i32, vp, _P(sz)]),
    "bitnet_decoder_read": (i32, [vp, i32, vp, sz]),
    "bitnet_allgather_output": (i32, [vp, sz, sz, sz, _P(vp), i32, sz, vp]),
    "bitnet_nccl_unique_id": (i32, [vp]),
    "bitnet_nccl_comm_create": (i32, [vp, i32, i32, _P(vp)]),
    "bitnet_nccl_comm_destroy": (i32, [vp]),
    "bitnet_allgather_output_nccl": (i32, [vp, vp, sz, sz, vp, vp, i32, sz, vp]),
    "bitnet_backend_pin_host": (i32, [vp, vp, sz]),
    "bitnet_backend_unpin_host": (i32, [vp, vp]),
    "bitnet_bitlinear_group_create": (i32, [_P(BitLinearGroupMember), sz, sz, sz, _P(vp)]),
    "bitnet_bitlinear_group_run": (i32, [vp, vp]),
    "bitnet_bitlinear_group_destroy": (None, [vp]),
    "bitnet_ffn_group_create": (i32, [_P(FfnGroupMember), sz, sz, sz, _P(vp)]),
    "bitnet_ffn_group_run": (i32, [vp, vp]),
    "bitnet_ffn_group_destroy": (None, [vp]),
    "bitnet_backend_ffn_plan_create": (i32, [vp, _P(FfnCall), sz, _P(ForwardOpts), sz, _P(vp)]),
    "bitnet_backend_ffn_plan_run": (i32, [vp]),
    "bitnet_backend_ffn_plan_destroy": (None, [vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library and attach the signatures; raises if it is not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m bitnet_mlx_rs_b200.build` "
                "(there is no fallback implementation)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)     # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().bitnet_last_error_string().decode("utf-8", "replace")
