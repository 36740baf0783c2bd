// TEST INFRASTRUCTURE.  The reference's projection forward kernel
// (src/kernels/projection/ProjectionFwd_kernel.cuh:15-153) for Vanilla3DGS<3>,
// PINHOLE, no distortion, launched on raw device buffers.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/projection/ProjectionFwd_kernel.cuh"
#include "ref_common.cuh"
#include "ref_sync.h"

extern "C" int ref_project_fwd(
    uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_stride,
    const float* viewmats, const float* intrins,
    float* aabb, float* depths, float* radii,
    float* xy, float* depth, float* conic, float* opac, float* rgb) {
    RawWorld world(N, means, quats, scales, opacities, dc, sh);
    RawScreen screen((int64_t)C * N, xy, depth, conic, opac, rgb);
    projection_fused_fwd_kernel_wrapper<RefPrim, CameraModelType::PINHOLE, CameraDistortionType::None>(
        0, C, N, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer((float*)nullptr), W, H,
        (float4*)aabb, depths, radii, screen, sh_packed, (const float2*)sh_bounds, 15, sh_bits, sh_stride);
    return ref_finish();
}
