// TEST INFRASTRUCTURE.  The reference's projection backward kernel
// (src/kernels/projection/ProjectionBwd_kernel.cuh:16-179) for Vanilla3DGS<3>,
// PINHOLE, no distortion, launched on raw device buffers.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/projection/ProjectionBwd_kernel.cuh"
#include "ref_common.cuh"
#include "ref_sync.h"

extern "C" int ref_project_bwd(
    uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_stride,
    const float* viewmats, const float* intrins, const float* aabb,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb,
    float* g_means, float* g_quats, float* g_scales, float* g_opacities, float* g_dc, float* g_sh) {
    RawWorld world(N, means, quats, scales, opacities, dc, sh);
    RawWorld grads(N, g_means, g_quats, g_scales, g_opacities, g_dc, g_sh);
    RawScreen v_screen((int64_t)C * N, v_xy, v_depth, v_conic, v_opac, v_rgb);
    projection_fused_bwd_kernel_wrapper<RefPrim, CameraModelType::PINHOLE, CameraDistortionType::None>(
        0, C, N, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer((float*)nullptr), W, H,
        nullptr, nullptr, (const float4*)aabb, v_screen, grads, nullptr,
        sh_packed, (const float2*)sh_bounds, 15, sh_bits, sh_stride);
    return ref_finish();
}
