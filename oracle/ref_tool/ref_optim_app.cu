// TEST INFRASTRUCTURE.  The reference's appearance Adam kernels
// (src/kernels/optim/FusedAppearanceOptim.cu:11-56 fp32, :291-418 doubly quantised),
// launched as fused_adam_step (:59-92) and fused_adam_step_quantized_value (:421-479) do.
#include "kernels/optim/FusedAppearanceOptim.cu"
#include "ref_sync.h"

extern "C" int ref_adam_plain(int64_t numel, int step, float lr, float l2_reg, float l2_reg_offset, float grad_scale, int zero_grad,
                              float* param, float* grad, float* exp_avg, float* exp_avg_sq) {
    auto kfn = zero_grad ? fused_adam_with_steps_kernel<true> : fused_adam_with_steps_kernel<false>;
    kfn<<<_CEIL_DIV((uint32_t)numel, 256), 256>>>(param, grad, exp_avg, exp_avg_sq, lr, step, nullptr, 2.0f * l2_reg / (float)numel, l2_reg_offset,
                                                 grad_scale, numel, 1);
    return ref_finish();
}

extern "C" int ref_adam_qq(int64_t numel, int step, float lr, float l2_reg, float grad_scale, int zero_grad, int value_bits,
                           float* grad, uint8_t* optim_packed, float* optim_bounds, uint8_t* value_packed, float* value_bounds) {
    const float decay = 2.0f * l2_reg / (float)numel;
    uint32_t blocks = _CEIL_DIV((uint32_t)numel, 256);
    #define ARGS grad, nullptr, nullptr, optim_packed, (float4*)optim_bounds, value_packed, (float2*)value_bounds, lr, step, nullptr, decay, 0.0f, grad_scale, numel, 45
    if (value_bits == 16) {
        if (zero_grad) fused_adam_with_steps_qq_kernel<256, 8, 16, true><<<blocks, 256>>>(ARGS);
        else fused_adam_with_steps_qq_kernel<256, 8, 16, false><<<blocks, 256>>>(ARGS);
    } else {
        if (zero_grad) fused_adam_with_steps_qq_kernel<256, 8, 8, true><<<blocks, 256>>>(ARGS);
        else fused_adam_with_steps_qq_kernel<256, 8, 8, false><<<blocks, 256>>>(ARGS);
    }
    #undef ARGS
    return ref_finish();
}

// fused_adam_step_quantized (:232-271): fp32 values, QuantizedAdamState<8,256> state.
extern "C" int ref_adam_q8(int64_t numel, int step, float lr, float l2_reg, float grad_scale, int zero_grad,
                           float* param, float* grad, uint8_t* optim_packed, float* optim_bounds) {
    const float decay = 2.0f * l2_reg / (float)numel;
    uint32_t blocks = _CEIL_DIV((uint32_t)numel, 256);
    if (zero_grad) fused_adam_with_steps_8bit_kernel<256, 8, true><<<blocks, 256>>>(param, grad, optim_packed, (float4*)optim_bounds, lr, step, nullptr, decay, 0.0f, grad_scale, numel, 45);
    else fused_adam_with_steps_8bit_kernel<256, 8, false><<<blocks, 256>>>(param, grad, optim_packed, (float4*)optim_bounds, lr, step, nullptr, decay, 0.0f, grad_scale, numel, 45);
    return ref_finish();
}

// The two kernels above with per-splat step counters, steps[idx / stride] (:34, :330).  The quantised kernel
// evaluates steps[idx / stride] for every thread of its last block, so `steps` must cover ceil(numel / 256) * 256 cells.
extern "C" int ref_adam_plain_steps(int64_t numel, const int32_t* steps, int stride, float lr, float l2_reg, float l2_reg_offset, float grad_scale,
                                    int zero_grad, float* param, float* grad, float* exp_avg, float* exp_avg_sq) {
    auto kfn = zero_grad ? fused_adam_with_steps_kernel<true> : fused_adam_with_steps_kernel<false>;
    kfn<<<_CEIL_DIV((uint32_t)numel, 256), 256>>>(param, grad, exp_avg, exp_avg_sq, lr, 1, steps, 2.0f * l2_reg / (float)numel, l2_reg_offset,
                                                 grad_scale, numel, stride);
    return ref_finish();
}

extern "C" int ref_adam_qq_steps(int64_t numel, const int32_t* steps, int stride, float lr, float l2_reg, float grad_scale, int zero_grad,
                                 int value_bits, float* grad, uint8_t* optim_packed, float* optim_bounds, uint8_t* value_packed,
                                 float* value_bounds) {
    const float decay = 2.0f * l2_reg / (float)numel;
    uint32_t blocks = _CEIL_DIV((uint32_t)numel, 256);
    #define ARGS grad, nullptr, nullptr, optim_packed, (float4*)optim_bounds, value_packed, (float2*)value_bounds, lr, 1, steps, decay, 0.0f, grad_scale, numel, stride
    if (value_bits == 16) {
        if (zero_grad) fused_adam_with_steps_qq_kernel<256, 8, 16, true><<<blocks, 256>>>(ARGS);
        else fused_adam_with_steps_qq_kernel<256, 8, 16, false><<<blocks, 256>>>(ARGS);
    } else {
        if (zero_grad) fused_adam_with_steps_qq_kernel<256, 8, 8, true><<<blocks, 256>>>(ARGS);
        else fused_adam_with_steps_qq_kernel<256, 8, 8, false><<<blocks, 256>>>(ARGS);
    }
    #undef ARGS
    return ref_finish();
}

// QuantizedAdamState<4,256> (one byte per cell): fused_adam_step_quantized with bits = 4 (:256-259) and
// fused_adam_step_quantized_value with optim_bits = 4 (:455-462).
extern "C" int ref_adam_q4(int64_t numel, int step, float lr, float l2_reg, float grad_scale, int zero_grad,
                           float* param, float* grad, uint8_t* optim_packed, float* optim_bounds) {
    const float decay = 2.0f * l2_reg / (float)numel;
    uint32_t blocks = _CEIL_DIV((uint32_t)numel, 256);
    if (zero_grad) fused_adam_with_steps_8bit_kernel<256, 4, true><<<blocks, 256>>>(param, grad, optim_packed, (float4*)optim_bounds, lr, step, nullptr, decay, 0.0f, grad_scale, numel, 45);
    else fused_adam_with_steps_8bit_kernel<256, 4, false><<<blocks, 256>>>(param, grad, optim_packed, (float4*)optim_bounds, lr, step, nullptr, decay, 0.0f, grad_scale, numel, 45);
    return ref_finish();
}

extern "C" int ref_adam_qq_o4(int64_t numel, int step, float lr, float l2_reg, float grad_scale, int zero_grad, int value_bits,
                              float* grad, uint8_t* optim_packed, float* optim_bounds, uint8_t* value_packed, float* value_bounds) {
    const float decay = 2.0f * l2_reg / (float)numel;
    uint32_t blocks = _CEIL_DIV((uint32_t)numel, 256);
    #define ARGS grad, nullptr, nullptr, optim_packed, (float4*)optim_bounds, value_packed, (float2*)value_bounds, lr, step, nullptr, decay, 0.0f, grad_scale, numel, 45
    if (value_bits == 16) {
        if (zero_grad) fused_adam_with_steps_qq_kernel<256, 4, 16, true><<<blocks, 256>>>(ARGS);
        else fused_adam_with_steps_qq_kernel<256, 4, 16, false><<<blocks, 256>>>(ARGS);
    } else {
        if (zero_grad) fused_adam_with_steps_qq_kernel<256, 4, 8, true><<<blocks, 256>>>(ARGS);
        else fused_adam_with_steps_qq_kernel<256, 4, 8, false><<<blocks, 256>>>(ARGS);
    }
    #undef ARGS
    return ref_finish();
}
