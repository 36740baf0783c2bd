// TEST INFRASTRUCTURE.  The reference's projection forward kernel
// (src/kernels/projection/ProjectionFwd_kernel.cuh:15-153) for Vanilla3DGS<3> with a lens-distortion tier, for the
// (camera model, tier) pairs of its instantiation table (src/kernels/projection/CameraVariants.cuh:11-22), launched on
// raw device buffers.  model: 0 = pinhole, 1 = fisheye, 2 = equisolid; tier: 1 = OpenCV, 2 = thin prism, 3 = rational
// (src/core/Common.cuh:94-109).  dist_coeffs: device [C][8].
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/projection/ProjectionFwd_kernel.cuh"
#include "ref_common.cuh"
#include "ref_sync.h"

template <CameraModelType MODEL, CameraDistortionType DIST>
static void run_fwd(uint32_t C, uint32_t N, uint32_t W, uint32_t H, RawWorld& world, const float* viewmats, const float* intrins, float* dist_coeffs,
                    float* aabb, float* depths, float* radii, RawScreen& screen) {
    projection_fused_fwd_kernel_wrapper<RefPrim, MODEL, DIST>(
        0, C, N, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer(dist_coeffs), W, H,
        (float4*)aabb, depths, radii, screen, nullptr, nullptr, 15, 32, 256);
}

extern "C" int ref_project_fwd_dist(
    int model, int tier, uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const float* viewmats, const float* intrins, float* dist_coeffs,
    float* aabb, float* depths, float* radii,
    float* xy, float* depth, float* conic, float* opac, float* rgb) {
    RawWorld world(N, means, quats, scales, opacities, dc, sh);
    RawScreen screen((int64_t)C * N, xy, depth, conic, opac, rgb);
#define RUN(M, D) run_fwd<CameraModelType::M, CameraDistortionType::D>(C, N, W, H, world, viewmats, intrins, dist_coeffs, aabb, depths, radii, screen)
    if (model == 0 && tier == 1) RUN(PINHOLE, OpenCV);
    else if (model == 0 && tier == 2) RUN(PINHOLE, ThinPrism);
    else if (model == 0 && tier == 3) RUN(PINHOLE, Rational);
    else if (model == 1 && tier == 1) RUN(FISHEYE, OpenCV);
    else if (model == 1 && tier == 2) RUN(FISHEYE, ThinPrism);
    else if (model == 2 && tier == 1) RUN(EQUISOLID, OpenCV);
    else if (model == 2 && tier == 2) RUN(EQUISOLID, ThinPrism);
    else return -1;
#undef RUN
    return ref_finish();
}
