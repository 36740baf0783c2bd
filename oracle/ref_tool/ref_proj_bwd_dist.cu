// TEST INFRASTRUCTURE.  The reference's projection backward kernel
// (src/kernels/projection/ProjectionBwd_kernel.cuh:16-179) for Vanilla3DGS<3> with a lens-distortion tier, for the
// (camera model, tier) pairs of its instantiation table (src/kernels/projection/CameraVariants.cuh:11-22), launched on
// raw device buffers.  model: 0 = pinhole, 1 = fisheye, 2 = equisolid; tier: 1 = OpenCV, 2 = thin prism, 3 = rational.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/projection/ProjectionBwd_kernel.cuh"
#include "ref_common.cuh"
#include "ref_sync.h"

template <CameraModelType MODEL, CameraDistortionType DIST>
static void run_bwd(uint32_t C, uint32_t N, uint32_t W, uint32_t H, RawWorld& world, const float* viewmats, const float* intrins, float* dist_coeffs,
                    const float* aabb, RawScreen& v_screen, RawWorld& grads) {
    projection_fused_bwd_kernel_wrapper<RefPrim, MODEL, DIST>(
        0, C, N, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer(dist_coeffs), W, H,
        nullptr, nullptr, (const float4*)aabb, v_screen, grads, nullptr, nullptr, nullptr, 15, 32, 256);
}

extern "C" int ref_project_bwd_dist(
    int model, int tier, uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const float* viewmats, const float* intrins, float* dist_coeffs, const float* aabb,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb,
    float* g_means, float* g_quats, float* g_scales, float* g_opacities, float* g_dc, float* g_sh) {
    RawWorld world(N, means, quats, scales, opacities, dc, sh);
    RawWorld grads(N, g_means, g_quats, g_scales, g_opacities, g_dc, g_sh);
    RawScreen v_screen((int64_t)C * N, v_xy, v_depth, v_conic, v_opac, v_rgb);
#define RUN(M, D) run_bwd<CameraModelType::M, CameraDistortionType::D>(C, N, W, H, world, viewmats, intrins, dist_coeffs, aabb, v_screen, grads)
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
