// TEST INFRASTRUCTURE.  The reference's fused geometry Adam kernel
// (src/kernels/optim/FusedGeometryOptim.cu:83-380), launched as
// fused_optim_3dgs_geometry does (:447-468), fp32 state.  ref_adam_geometry: every regulariser
// weight zero, no scale-agnostic mean, scalar step; ref_adam_geometry_ex: those three switched on.
#include "kernels/optim/FusedGeometryOptim.cu"
#include "ref_sync.h"

extern "C" int ref_adam_geometry(
    int64_t N, int step, float grad_scale, int zero_grad, float lr_means, float lr_quats, float lr_scales, float lr_opacs,
    float* means, float* v_means, float* g1_means, float* g2_means,
    float* quats, float* v_quats, float* g1_quats, float* g2_quats,
    float* scales, float* v_scales, float* g1_scales, float* g2_scales,
    float* opacs, float* v_opacs, float* g1_opacs, float* g2_opacs) {
    NonShQuantState non_sh;
    GradQuantBuffers gq;
    auto launch = [&](auto kfn) {
        kfn<<<_CEIL_DIV((uint32_t)N, 256), 256>>>(
            (float3*)means, (float3*)v_means, (float3*)g1_means, (float3*)g2_means,
            (float4*)quats, (float4*)v_quats, (float4*)g1_quats, (float4*)g2_quats,
            (float3*)scales, (float3*)v_scales, (float3*)g1_scales, (float3*)g2_scales,
            opacs, v_opacs, g1_opacs, g2_opacs,
            nullptr, nullptr, nullptr, nullptr,
            lr_means, lr_quats, lr_scales, lr_opacs, 0.0f,
            0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, grad_scale,
            non_sh, gq, step, nullptr, N);
    };
    if (zero_grad) launch(fused_optim_3dgs_geometry_kernel<false, true, false>);
    else launch(fused_optim_3dgs_geometry_kernel<false, false, false>);
    return ref_finish();
}

// reg = max_gauss_ratio, scale_regularization, mcmc_opacity, mcmc_scale, erank, erank_s3, quat_norm (undivided,
// the division by N is the launcher's, :457-462); radii and steps may be null.
extern "C" int ref_adam_geometry_ex(
    int64_t N, int step, float grad_scale, int zero_grad, float lr_means, float lr_quats, float lr_scales, float lr_opacs,
    float* means, float* v_means, float* g1_means, float* g2_means,
    float* quats, float* v_quats, float* g1_quats, float* g2_quats,
    float* scales, float* v_scales, float* g1_scales, float* g2_scales,
    float* opacs, float* v_opacs, float* g1_opacs, float* g2_opacs,
    const float* reg, int use_scale_agnostic_mean, const float* radii, const int32_t* steps, float* densify_score) {
    NonShQuantState non_sh;
    GradQuantBuffers gq;
    const float n = (float)N;
    auto launch = [&](auto kfn) {
        kfn<<<_CEIL_DIV((uint32_t)N, 256), 256>>>(
            (float3*)means, (float3*)v_means, (float3*)g1_means, (float3*)g2_means,
            (float4*)quats, (float4*)v_quats, (float4*)g1_quats, (float4*)g2_quats,
            (float3*)scales, (float3*)v_scales, (float3*)g1_scales, (float3*)g2_scales,
            opacs, v_opacs, g1_opacs, g2_opacs,
            nullptr, nullptr, radii, densify_score,
            lr_means, lr_quats, lr_scales, lr_opacs, 0.0f,
            reg[0], reg[1] / n, reg[2] / n, reg[3] / n, reg[4] / n, reg[5] / n, reg[6] / n, 0.0f, grad_scale,
            non_sh, gq, step, steps, N);
    };
    if (use_scale_agnostic_mean) {
        if (zero_grad) launch(fused_optim_3dgs_geometry_kernel<true, true, false>);
        else launch(fused_optim_3dgs_geometry_kernel<true, false, false>);
    } else {
        if (zero_grad) launch(fused_optim_3dgs_geometry_kernel<false, true, false>);
        else launch(fused_optim_3dgs_geometry_kernel<false, false, false>);
    }
    return ref_finish();
}


// The non_sh_quant instantiation (moments of all five arrays in 16-bit joint codes, one float4 of bounds per 256 splats and
// array; DC updated in the same kernel): FusedGeometryOptim.cu:144-380.  packed / bounds: means, quats, scales, opacities, dc.
extern "C" int ref_adam_geometry_q16(
    int64_t N, int step, float grad_scale, int zero_grad, float lr_means, float lr_quats, float lr_scales, float lr_opacs, float lr_dc, float sh_reg_weight,
    float* means, float* v_means, float* quats, float* v_quats, float* scales, float* v_scales, float* opacs, float* v_opacs, float* dc, float* v_dc,
    uint8_t* const* packed, float* const* bounds, const float* reg, const int32_t* steps) {
    NonShQuantState non_sh;
    non_sh.enabled = true;
    non_sh.means_packed = packed[0]; non_sh.quats_packed = packed[1]; non_sh.scales_packed = packed[2]; non_sh.opacities_packed = packed[3];
    non_sh.features_dc_packed = packed[4];
    non_sh.means_bounds = (float4*)bounds[0]; non_sh.quats_bounds = (float4*)bounds[1]; non_sh.scales_bounds = (float4*)bounds[2];
    non_sh.opacities_bounds = (float4*)bounds[3]; non_sh.features_dc_bounds = (float4*)bounds[4];
    GradQuantBuffers gq;
    const float zero7[7] = {0, 0, 0, 0, 0, 0, 0};
    const float* r = reg ? reg : zero7;
    const float n = (float)N;      // the weights arrive undivided, as in ref_adam_geometry_ex
    auto launch = [&](auto kfn) {
        kfn<<<_CEIL_DIV((uint32_t)N, 256), 256>>>(
            (float3*)means, (float3*)v_means, nullptr, nullptr, (float4*)quats, (float4*)v_quats, nullptr, nullptr,
            (float3*)scales, (float3*)v_scales, nullptr, nullptr, opacs, v_opacs, nullptr, nullptr,
            (float3*)dc, (float3*)v_dc, nullptr, nullptr,
            lr_means, lr_quats, lr_scales, lr_opacs, lr_dc,
            r[0], r[1] / n, r[2] / n, r[3] / n, r[4] / n, r[5] / n, r[6] / n, sh_reg_weight, grad_scale,
            non_sh, gq, step, steps, N);
    };
    if (zero_grad) launch(fused_optim_3dgs_geometry_kernel<false, true, true>);
    else launch(fused_optim_3dgs_geometry_kernel<false, false, true>);
    return ref_finish();
}
