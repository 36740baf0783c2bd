// TEST INFRASTRUCTURE.  The reference's fused geometry Adam kernel
// (src/kernels/optim/FusedGeometryOptim.cu:83-380), launched as
// fused_optim_3dgs_geometry does (:447-468) with every regulariser weight zero,
// fp32 state, no scale-agnostic mean, scalar step.
#include "kernels/optim/FusedGeometryOptim.cu"

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
    return (int)cudaDeviceSynchronize();
}
