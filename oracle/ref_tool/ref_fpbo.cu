// TEST INFRASTRUCTURE.  The reference's fused projection-backward + optimiser kernel
// (src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:146-1140) for Vanilla3DGS<3>, PINHOLE, no distortion, quantisation
// level 0 (fp32 values and moments), launched on raw device buffers.  aabb and the screen gradients are indexed
// [view][splat]; the kernel runs in its packed mode (the reference's stock mode) over an index that lists every
// (view, splat) pair: bounds[g] = g*C, perm[g*C + c] = c*N + g, camera_ids[c*N + g] = c.  The unpacked mode is not used
// because the threads past N of the last block would run the view loop there on unloaded splats (cid_1 stays C for them).
// reg: max_gauss_ratio and the six undivided regulariser weights; the wrapper divides them by N itself.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/optim/FusedProjectionBwdOptim_kernel.cuh"
#include "ref_common.cuh"
#include "ref_sync.h"
#include <vector>

template <bool AGNOSTIC>
static void run_fpbo(uint32_t C, uint32_t N, uint32_t W, uint32_t H, RawWorld& world, const float* viewmats, const float* intrins, const int32_t* index, const float* aabb,
                     RawWorld& v_world, RawScreen& v_screen, RawWorld& g1, RawWorld& g2, const float* radii, const float* lrs, const float* reg,
                     float sh_reg_weight, int step, const int32_t* steps) {
    NonShQuantState non_sh;
    fused_projection_bwd_optimizer_3dgs_kernel_wrapper<RefPrim, CameraModelType::PINHOLE, CameraDistortionType::None, AGNOSTIC, false, 0>(
        0, C, N, 15, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer((float*)nullptr), W, H,
        index, index + (N + 1), index + (N + 1) + (size_t)C * N, (const float4*)aabb, v_world, v_screen, g1, g2, nullptr, nullptr, nullptr, nullptr, non_sh,
        radii, nullptr, lrs[0], lrs[1], lrs[2], lrs[3], lrs[4], lrs[5],
        reg[0], reg[1], reg[2], reg[3], reg[4], reg[5], reg[6], sh_reg_weight, 0.0f, step, steps);
}

extern "C" int ref_fpbo(
    uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const float* viewmats, const float* intrins, const float* aabb,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb,
    float* z_means, float* z_quats, float* z_scales, float* z_opacities, float* z_dc, float* z_sh,          // zeroed world-gradient arrays
    float* g1_means, float* g1_quats, float* g1_scales, float* g1_opacities, float* g1_dc, float* g1_sh,
    float* g2_means, float* g2_quats, float* g2_scales, float* g2_opacities, float* g2_dc, float* g2_sh,
    const float* radii, const float* lrs, const float* reg, float sh_reg_weight, int use_scale_agnostic_mean, int step, const int32_t* steps) {
    RawWorld world(N, means, quats, scales, opacities, dc, sh);
    RawWorld v_world(N, z_means, z_quats, z_scales, z_opacities, z_dc, z_sh);
    RawWorld g1(N, g1_means, g1_quats, g1_scales, g1_opacities, g1_dc, g1_sh);
    RawWorld g2(N, g2_means, g2_quats, g2_scales, g2_opacities, g2_dc, g2_sh);
    RawScreen v_screen((int64_t)C * N, v_xy, v_depth, v_conic, v_opac, v_rgb);
    std::vector<int32_t> h((size_t)N + 1 + 2 * (size_t)C * N);
    int32_t *bounds = h.data(), *cam = bounds + N + 1, *perm = cam + (size_t)C * N;
    for (uint32_t g = 0; g <= N; ++g) bounds[g] = (int32_t)(g * C);
    for (uint32_t c = 0; c < C; ++c)
        for (uint32_t g = 0; g < N; ++g) { cam[(size_t)c * N + g] = (int32_t)c; perm[(size_t)g * C + c] = (int32_t)(c * N + g); }
    int32_t* index = nullptr;
    if (cudaMalloc(&index, h.size() * sizeof(int32_t)) != cudaSuccess) return (int)cudaGetLastError();
    cudaMemcpy(index, h.data(), h.size() * sizeof(int32_t), cudaMemcpyHostToDevice);
    if (use_scale_agnostic_mean) run_fpbo<true>(C, N, W, H, world, viewmats, intrins, index, aabb, v_world, v_screen, g1, g2, radii, lrs, reg, sh_reg_weight, step, steps);
    else run_fpbo<false>(C, N, W, H, world, viewmats, intrins, index, aabb, v_world, v_screen, g1, g2, radii, lrs, reg, sh_reg_weight, step, steps);
    const int rc = (int)cudaDeviceSynchronize();
    cudaFree(index);
    return rc;
}
