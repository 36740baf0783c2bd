// TEST INFRASTRUCTURE.  The reference's projection forward and backward kernels
// (src/kernels/projection/ProjectionFwd_kernel.cuh:15-153, ProjectionBwd_kernel.cuh:16-179) for Vanilla3DGS<0>, <1> and
// <2> -- the instantiations its trainer uses while the SH degree is warmed up (sh_degree_to_use,
// src/app/TrainerCore.cpp:948) -- PINHOLE, no distortion, on raw device buffers.  The SH array keeps its 15-coefficient
// rows (stride 45), as the engine's does; a lower degree reads only the leading coefficients of a row.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/projection/ProjectionFwd_kernel.cuh"
#include "kernels/projection/ProjectionBwd_kernel.cuh"
#include "ref_sync.h"

template <class Prim>
struct RawWorldT : Prim::WorldBuffer {
    RawWorldT(int64_t n, float* means, float* quats, float* scales, float* opacities, float* dc, float* sh) {
        this->_size = n;
        float* p[6] = {means, quats, scales, opacities, dc, sh};
        int32_t st[6] = {3, 4, 3, 1, 3, 45};
        for (int i = 0; i < 6; ++i) { this->_data[i] = p[i]; this->_strides[i] = st[i]; }
    }
};
template <class Prim>
struct RawScreenT : Prim::ScreenBuffer {
    RawScreenT(int64_t n, float* xy, float* depth, float* conic, float* opac, float* rgb) {
        this->_size = n;
        float* p[5] = {xy, depth, conic, opac, rgb};
        int32_t st[5] = {2, 1, 3, 1, 3};
        for (int i = 0; i < 5; ++i) { this->_data[i] = p[i]; this->_strides[i] = st[i]; }
    }
};

template <int DEG>
static void run_fwd(uint32_t C, uint32_t N, uint32_t W, uint32_t H, float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
                    const float* viewmats, const float* intrins, float* aabb, float* depths, float* radii,
                    float* xy, float* depth, float* conic, float* opac, float* rgb) {
    typedef Vanilla3DGS<DEG> Prim;
    RawWorldT<Prim> world(N, means, quats, scales, opacities, dc, sh);
    RawScreenT<Prim> screen((int64_t)C * N, xy, depth, conic, opac, rgb);
    projection_fused_fwd_kernel_wrapper<Prim, CameraModelType::PINHOLE, CameraDistortionType::None>(
        0, C, N, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer((float*)nullptr), W, H,
        (float4*)aabb, depths, radii, screen, nullptr, nullptr, 15, 32, 256);
}

extern "C" int ref_project_fwd_deg(
    int degree, uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const float* viewmats, const float* intrins, float* aabb, float* depths, float* radii,
    float* xy, float* depth, float* conic, float* opac, float* rgb) {
    if (degree == 0) run_fwd<0>(C, N, W, H, means, quats, scales, opacities, dc, sh, viewmats, intrins, aabb, depths, radii, xy, depth, conic, opac, rgb);
    else if (degree == 1) run_fwd<1>(C, N, W, H, means, quats, scales, opacities, dc, sh, viewmats, intrins, aabb, depths, radii, xy, depth, conic, opac, rgb);
    else if (degree == 2) run_fwd<2>(C, N, W, H, means, quats, scales, opacities, dc, sh, viewmats, intrins, aabb, depths, radii, xy, depth, conic, opac, rgb);
    else return -1;
    return ref_finish();
}

template <int DEG>
static void run_bwd(uint32_t C, uint32_t N, uint32_t W, uint32_t H, float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
                    const float* viewmats, const float* intrins, const float* aabb,
                    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb,
                    float* g_means, float* g_quats, float* g_scales, float* g_opacities, float* g_dc, float* g_sh) {
    typedef Vanilla3DGS<DEG> Prim;
    RawWorldT<Prim> world(N, means, quats, scales, opacities, dc, sh);
    RawWorldT<Prim> grads(N, g_means, g_quats, g_scales, g_opacities, g_dc, g_sh);
    RawScreenT<Prim> v_screen((int64_t)C * N, v_xy, v_depth, v_conic, v_opac, v_rgb);
    projection_fused_bwd_kernel_wrapper<Prim, CameraModelType::PINHOLE, CameraDistortionType::None>(
        0, C, N, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer((float*)nullptr), W, H,
        nullptr, nullptr, (const float4*)aabb, v_screen, grads, nullptr, nullptr, nullptr, 15, 32, 256);
}

extern "C" int ref_project_bwd_deg(
    int degree, uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const float* viewmats, const float* intrins, const float* aabb,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb,
    float* g_means, float* g_quats, float* g_scales, float* g_opacities, float* g_dc, float* g_sh) {
#define RUN(D) run_bwd<D>(C, N, W, H, means, quats, scales, opacities, dc, sh, viewmats, intrins, aabb, v_xy, v_depth, v_conic, v_opac, v_rgb, \
                          g_means, g_quats, g_scales, g_opacities, g_dc, g_sh)
    if (degree == 0) RUN(0);
    else if (degree == 1) RUN(1);
    else if (degree == 2) RUN(2);
    else return -1;
#undef RUN
    return ref_finish();
}
