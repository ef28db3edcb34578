// Exported placeholders for the part of the reference's symbol list that lies outside the
// quantized-decode path (dense GEMM, attention, convolution, training ops, the TCP collectives,
// DiLoCo, checkpointing, memory tiers, HIP, the Eshkol bridge).  The reference's ctypes binding
// resolves every exported name when it is imported, so each must exist; none of them computes
// anything here.  Status-returning entry points answer TC_ERR_UNSUPPORTED_FAMILY (-4), counters
// answer 0, pointers and strings answer NULL / "unsupported".  On x86-64 and AArch64 a callee
// that ignores its arguments is ABI-compatible with any argument list the caller pushes.
#include <stdint.h>

#define TCB_UNSUPPORTED (-4)
#define TCB_EXPORT extern "C" __attribute__((visibility("default")))

TCB_EXPORT int tc_adamw_step(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_attention_backward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_buffer_demote_async(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_buffer_get_tier(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_buffer_promote_async(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_buffer_set_tier_hint(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_buffer_tier_sync(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_checkpoint_discard(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_checkpoint_realize(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_checkpoint_register(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_checkpoint_unregister(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_conv2d_backward_input(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_conv2d_backward_weight(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_conv2d_forward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_diloco_add_parameter(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_diloco_apply_outer(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_diloco_finalize(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_diloco_init(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_diloco_step(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_hip_device_at(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_hip_device_info_get(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_hip_init(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_hip_select_device(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_layernorm_backward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_memory_tier_usage(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_rmsnorm_backward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_rope_backward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_softmax_backward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_softmax_forward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int tc_swiglu_backward(void) { return TCB_UNSUPPORTED; }

TCB_EXPORT int32_t tc_eshkol_attention_forward(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int32_t tc_eshkol_buffer_free(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int32_t tc_eshkol_gemm(void) { return TCB_UNSUPPORTED; }
TCB_EXPORT int32_t tc_eshkol_shutdown(void) { return TCB_UNSUPPORTED; }

TCB_EXPORT uint64_t tc_checkpoint_count_discarded(void) { return 0; }
TCB_EXPORT uint64_t tc_checkpoint_count_resident(void) { return 0; }
TCB_EXPORT uint64_t tc_checkpoint_total_bytes_discarded(void) { return 0; }
TCB_EXPORT uint64_t tc_diloco_inner_steps_completed(void) { return 0; }
TCB_EXPORT uint64_t tc_diloco_outer_steps_completed(void) { return 0; }
TCB_EXPORT int tc_checkpoint_is_resident(void) { return 0; }
TCB_EXPORT int tc_hip_device_count(void) { return 0; }
TCB_EXPORT int tc_eshkol_device_family(void) { return 0; }
TCB_EXPORT int tc_eshkol_device_supports_bf16(void) { return 0; }
TCB_EXPORT int tc_eshkol_device_supports_i8(void) { return 0; }
TCB_EXPORT int tc_eshkol_device_supports_tensorops_m5(void) { return 0; }
TCB_EXPORT int tc_eshkol_device_unified_memory(void) { return 0; }
TCB_EXPORT int tc_eshkol_last_backend_code(void) { return 0; }
TCB_EXPORT double tc_diloco_last_outer_bytes_sent(void) { return 0.0; }
TCB_EXPORT double tc_diloco_last_outer_step_seconds(void) { return 0.0; }
TCB_EXPORT void* tc_eshkol_buffer_alloc(void) { return nullptr; }
TCB_EXPORT void* tc_eshkol_buffer_map(void) { return nullptr; }
TCB_EXPORT void* tc_eshkol_init(void) { return nullptr; }
TCB_EXPORT const char* tc_eshkol_device_name(void) { return "unsupported"; }
TCB_EXPORT const char* tc_eshkol_last_backend(void) { return "unsupported"; }
TCB_EXPORT const char* tc_eshkol_status_string(void) { return "unsupported"; }
TCB_EXPORT const char* tc_eshkol_version(void) { return "unsupported"; }
TCB_EXPORT const char* tc_hip_last_kernel_name(void) { return "unsupported"; }

// include/tensorcore/gemm.h: returns NULL and reports the reason through *err.
TCB_EXPORT const char* tc_tensorops_gemm_kernel_name(const void* desc, int* err) {
    (void)desc;
    if (err) *err = -5;  // TC_ERR_UNSUPPORTED_DTYPE
    return nullptr;
}
