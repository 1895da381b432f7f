"""ctypes binding of libfe2o3_b200.so (the C ABI declared in include/fe2o3_b200.h).

There is no CPU fallback: if the shared library is missing, importing this
module raises.  Build it with `python fe2o3_b200/build.py`.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FE2O3_B200_LIB names another build of the same library (for instance one compiled with diagnostics)
LIB_PATH = os.environ.get("FE2O3_B200_LIB") or os.path.join(_HERE, "libfe2o3_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: the CUDA library must be built (python fe2o3_b200/build.py); "
        "fe2o3_b200 has no CPU fallback")

lib = C.CDLL(LIB_PATH)

u32, u64, i32, f32 = C.c_uint32, C.c_uint64, C.c_int32, C.c_float
vp = C.c_void_p


class Slice(C.Structure):
    _fields_ = [("ptr", u64), ("len", u64)]


def _struct(name, slices, scalars=()):
    fields = [(s, Slice) for s in slices] + list(scalars)
    return type(name, (C.Structure,), {"_fields_": fields})


ScalarGemmArgs = _struct("ScalarGemmArgs", ["a", "b", "c"], [("m", u32), ("n", u32), ("k", u32), ("reserved", u32)])
TiledGemmArgs = _struct("TiledGemmArgs", ["a", "b", "c"], [("m", u32), ("n", u32), ("k", u32), ("reserved", u32)])
TiledGemmGeneralArgs = _struct("TiledGemmGeneralArgs", ["a", "b", "c"],
                               [("m", u32), ("n", u32), ("k", u32), ("lda", u32), ("ldb", u32), ("ldc", u32),
                                ("alpha", f32), ("beta", f32)])
FlashAttentionArgs = _struct("FlashAttentionArgs", ["q", "k", "v", "output"],
                             [("batch", u32), ("heads", u32), ("seq", u32), ("dim", u32), ("scale", f32),
                              ("causal", u32), ("input_dtype", u32), ("reserved", u32)])
RowSoftmaxArgs = _struct("RowSoftmaxArgs", ["input", "output", "mask"], [("rows", u32), ("cols", u32)])
MoeTop2Args = _struct("MoeTop2Args", ["logits", "top2_experts", "requested_counts", "admitted_counts",
                                      "expert_offsets", "route_slots", "permutation", "inverse"],
                      [("tokens", u32), ("experts", u32), ("capacity", u32), ("reserved", u32)])
MoeGateArgs = _struct("MoeGateArgs", ["x", "wg", "logits"],
                      [("tokens", u32), ("d_model", u32), ("experts", u32), ("reserved", u32)])
MoeRouteWeightsArgs = _struct("MoeRouteWeightsArgs", ["logits", "top2_experts", "route_weights"],
                              [("tokens", u32), ("experts", u32)])
MoeExpertFfnArgs = _struct("MoeExpertFfnArgs", ["x", "w1", "w2", "permutation", "expert_offsets", "compact_x",
                                                "hidden", "compact_output"],
                           [("tokens", u32), ("d_model", u32), ("d_ff", u32), ("experts", u32)])
MoeCombineArgs = _struct("MoeCombineArgs", ["compact_output", "inverse", "route_weights", "combined_output"],
                         [("tokens", u32), ("width", u32)])
MoeExpertFfnCombineArgs = _struct("MoeExpertFfnCombineArgs", ["x", "w1", "w2", "permutation", "expert_offsets",
                                                              "route_weights", "hidden", "combined_output"],
                                  [("tokens", u32), ("d_model", u32), ("d_ff", u32), ("experts", u32)])
MoeCompactArgs = _struct("MoeCompactArgs", ["x", "permutation", "compact_x"], [("tokens", u32), ("d_model", u32)])
MoeGroupedFfnArgs = _struct("MoeGroupedFfnArgs", ["compact_x", "w1", "w2", "group_offsets", "hidden", "compact_output"],
                            [("d_model", u32), ("d_ff", u32), ("groups", u32), ("experts_cycle", u32)])
MoeEpExchangeArgs = _struct("MoeEpExchangeArgs",
                            ["x", "top2_experts", "permutation", "inverse", "expert_offsets", "admitted_counts",
                             "route_weights", "pair_offsets", "combined_output", "peer_recv_x", "peer_recv_meta",
                             "peer_ret", "peer_counts", "peer_flags", "epoch_counter", "logits"],
                            [("tokens", u32), ("d_model", u32), ("experts", u32), ("world", u32), ("rank", u32),
                             ("epoch", u32), ("max_rows", u32), ("phase", u32), ("spin_limit", u32), ("reserved", u32)])
MoeEpFfnArgs = _struct("MoeEpFfnArgs",
                       ["recv_x", "w1", "w2", "pair_offsets", "hidden", "recv_meta", "flags", "peer_ret", "peer_flags",
                        "epoch_counter", "progress"],
                       [("tokens", u32), ("d_model", u32), ("d_ff", u32), ("experts", u32), ("world", u32), ("rank", u32),
                        ("epoch", u32), ("max_rows", u32), ("spin_limit", u32), ("reserved", u32)])
MaskedReduceArgs = _struct("MaskedReduceArgs", ["values", "active", "output"])
MaskedReducePackedArgs = _struct("MaskedReducePackedArgs", ["values", "mask", "output"])
DeviceScanArgs = _struct("DeviceScanArgs", ["values", "output"], [("exclusive", u32), ("reserved", u32)])
WaveLdsArgs = _struct("WaveLdsArgs", ["values", "active", "wave_out", "workgroup_out"])


class Wave64CollectivesArgs(C.Structure):
    _fields_ = [("input", Slice), ("active_mask", u64), ("reduction_output", Slice), ("inclusive_output", Slice),
                ("exclusive_output", Slice)]


Wave64SegmentedArgs = _struct("Wave64SegmentedArgs", ["input", "masks", "reduction_output", "inclusive_output",
                                                      "exclusive_output"])
LdsReduceArgs = _struct("LdsReduceArgs", ["values", "output"])


class ScopedAtomicAddArgs(C.Structure):
    _fields_ = [("values", Slice), ("eligible", Slice), ("target", u64)]


class Geometry(C.Structure):
    _fields_ = [("grid", u32 * 3), ("workgroup", u32 * 3), ("dynamic_shared_bytes", u32), ("launches", u32)]


class HostCopy(C.Structure):
    _fields_ = [("buffer", vp), ("host", vp), ("elements", u64)]


class KernelResources(C.Structure):
    _fields_ = [("registers_per_thread", u32), ("static_shared_bytes", u32), ("max_dynamic_shared_bytes", u32),
                ("max_threads_per_block", u32), ("local_bytes_per_thread", u32), ("const_bytes", u32)]


class DeviceProperties(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("total_global_bytes", u64), ("compute_major", u32), ("compute_minor", u32),
                ("multiprocessors", u32), ("max_shared_bytes_per_block_optin", u32), ("l2_bytes", u32),
                ("sm_clock_khz", u32), ("mem_clock_khz", u32), ("warp_size", u32)]


# op name -> (args struct, kernarg bytes the reference-style block must have, takes schedule)
OPS = {
    "scalar_gemm_v1": (ScalarGemmArgs, 64, True),
    "tiled_gemm_v1": (TiledGemmArgs, 64, True),
    "tiled_gemm_general_v1": (TiledGemmGeneralArgs, 80, True),
    "flash_attention_v1": (FlashAttentionArgs, 96, False),
    "row_softmax_v1": (RowSoftmaxArgs, 56, False),
    "moe_top2_v1": (MoeTop2Args, 144, False),
    "moe_gate_v1": (MoeGateArgs, 64, False),
    "moe_route_weights_v1": (MoeRouteWeightsArgs, 56, False),
    "moe_expert_ffn_v1": (MoeExpertFfnArgs, 144, False),
    "moe_expert_combine_v1": (MoeCombineArgs, 72, False),
    "moe_compact_v1": (MoeCompactArgs, 56, False),
    "moe_grouped_ffn_v1": (MoeGroupedFfnArgs, 112, False),
    "moe_expert_ffn_combine_v1": (MoeExpertFfnCombineArgs, 144, False),
    "moe_ep_exchange_v1": (MoeEpExchangeArgs, 296, False),
    "moe_ep_ffn_v1": (MoeEpFfnArgs, 216, False),
    "masked_reduce_u32": (MaskedReduceArgs, 48, False),
    "masked_reduce_u32_packed": (MaskedReducePackedArgs, 48, False),
    "device_scan_u32": (DeviceScanArgs, 40, False),
    "device_scan_f32": (DeviceScanArgs, 40, False),
    "wave_lds_v1": (WaveLdsArgs, 64, False),
    "wave64_collectives_v1": (Wave64CollectivesArgs, 72, False),
    "wave64_collectives_segmented": (Wave64SegmentedArgs, 80, False),
    "lds_publish_read_reduce_i32_v1": (LdsReduceArgs, 32, False),
    "scoped_atomic_add_u32_v1": (ScopedAtomicAddArgs, 40, False),
}

# every exported symbol of include/fe2o3_b200.h
EXPORTS = [
    "fe2o3_ctx_create", "fe2o3_ctx_destroy", "fe2o3_ctx_bind_to_thread", "fe2o3_ctx_device",
    "fe2o3_ctx_observe_environment", "fe2o3_stream_default", "fe2o3_stream_create", "fe2o3_stream_sync",
    "fe2o3_stream_destroy", "fe2o3_stream_native", "fe2o3_stream_wrap", "fe2o3_buf_alloc_zeroed",
    "fe2o3_buf_from_host", "fe2o3_buf_to_host", "fe2o3_buf_copy_from_host_async", "fe2o3_buf_copy_to_host_async",
    "fe2o3_buf_free", "fe2o3_buf_quarantine", "fe2o3_buf_ptr", "fe2o3_buf_len", "fe2o3_buf_slice",
    "fe2o3_pinned_alloc", "fe2o3_pinned_free", "fe2o3_event_create", "fe2o3_event_record", "fe2o3_event_sync",
    "fe2o3_event_query", "fe2o3_event_elapsed_ms", "fe2o3_event_destroy", "fe2o3_stream_wait_event", "fe2o3_peer_access_enable",
    "fe2o3_status_string", "fe2o3_last_error", "fe2o3_prepared_launch", "fe2o3_prepared_launch_and_wait",
    "fe2o3_prepared_geometry", "fe2o3_prepared_kernarg", "fe2o3_prepared_patch_kernarg", "fe2o3_prepared_symbol", "fe2o3_prepared_destroy",
    "fe2o3_ctx_take_kernel_status", "fe2o3_load_executable", "fe2o3_resolve_kernel", "fe2o3_launch_and_wait",
    "fe2o3_image_digest", "fe2o3_observe_kernel_resources", "fe2o3_operation_submit", "fe2o3_operation_is_complete",
    "fe2o3_operation_wait", "fe2o3_operation_abandon",
    "fe2o3_unload_executable", "fe2o3_synth_uniform_f32", "fe2o3_synth_normal_f32", "fe2o3_synth_normal_bf16",
    "fe2o3_synth_uniform_bf16", "fe2o3_synth_u32_below", "fe2o3_synth_bernoulli", "fe2o3_synth_gemm_inputs_v1",
    "fe2o3_bf16_from_f32", "fe2o3_launch_count", "fe2o3_masked_reduce_u32_noalloc",
    "fe2o3_peer_region_create", "fe2o3_peer_region_export", "fe2o3_peer_region_import", "fe2o3_peer_region_ptr",
    "fe2o3_peer_region_bytes", "fe2o3_peer_region_destroy",
] + [f"fe2o3_{op}_check" for op in OPS] + [f"fe2o3_{op}_prepare" for op in OPS]

lib.fe2o3_status_string.restype = C.c_char_p
lib.fe2o3_status_string.argtypes = [i32]
lib.fe2o3_last_error.restype = C.c_char_p
lib.fe2o3_prepared_symbol.restype = C.c_char_p
lib.fe2o3_prepared_symbol.argtypes = [vp]
lib.fe2o3_buf_ptr.restype = u64
lib.fe2o3_buf_ptr.argtypes = [vp]
lib.fe2o3_buf_len.restype = u64
lib.fe2o3_buf_len.argtypes = [vp]
lib.fe2o3_launch_count.restype = u64
lib.fe2o3_peer_region_ptr.restype = u64
lib.fe2o3_peer_region_ptr.argtypes = [vp]
lib.fe2o3_peer_region_bytes.restype = u64
lib.fe2o3_peer_region_bytes.argtypes = [vp]
lib.fe2o3_bf16_from_f32.restype = C.c_uint16
lib.fe2o3_bf16_from_f32.argtypes = [f32]
for _n in EXPORTS:
    _f = getattr(lib, _n)
    if _f.restype is C.c_int:
        _f.restype = i32


class Fe2o3Error(RuntimeError):
    def __init__(self, status, where=""):
        self.status = int(status)
        self.name = lib.fe2o3_status_string(self.status).decode()
        self.detail = lib.fe2o3_last_error().decode()
        super().__init__(f"{where}: {self.name} ({self.status}): {self.detail}")


def check(status, where=""):
    if status != 0:
        raise Fe2o3Error(status, where)
