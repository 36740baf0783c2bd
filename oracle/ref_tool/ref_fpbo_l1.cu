// TEST INFRASTRUCTURE.  The reference's fused projection-backward + optimiser kernel at quantisation level 1
// (src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:146-1140: 16-bit SH values and 8-bit joint SH optimiser state with one
// bound per 256 splats; the moments of the five other arrays fp32 or, with nq_packed given, 16-bit codes) for Vanilla3DGS<3> and,
// for the SH degree warm-up, Vanilla3DGS<1> on the same 15-coefficient buffers; PINHOLE, no distortion, raw device buffers.
// Pointer groups are host arrays of device pointers: world6 = means, quats, scales, opacities, features_dc, features_sh (fp32,
// not read at this level); v_screen5 = xy, depth, conic, opacity, rgb; zero6 = zeroed world-gradient arrays; g1_5 / g2_5 = fp32
// moments of the five non-SH arrays (read when nq_packed is NULL).  The kernel runs in its packed mode over an index that
// lists every (view, splat) pair, as in ref_fpbo.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/optim/FusedProjectionBwdOptim_kernel.cuh"
#include "ref_sync.h"
#include <vector>

template <class Prim>
struct L1World : Prim::WorldBuffer {
    L1World(int64_t n, float* const* p) {
        this->_size = n;
        int32_t st[6] = {3, 4, 3, 1, 3, 45};
        for (int i = 0; i < 6; ++i) { this->_data[i] = p[i]; this->_strides[i] = st[i]; }
    }
};
template <class Prim>
struct L1Screen : Prim::ScreenBuffer {
    L1Screen(int64_t n, float* const* p) {
        this->_size = n;
        int32_t st[5] = {2, 1, 3, 1, 3};
        for (int i = 0; i < 5; ++i) { this->_data[i] = p[i]; this->_strides[i] = st[i]; }
    }
};

template <int DEG, bool AGNOSTIC>
static void run_l1(uint32_t C, uint32_t N, uint32_t W, uint32_t H, float* const* world6, const float* viewmats, const float* intrins, const int32_t* index,
                   const float* aabb, float* const* v_screen5, float* const* zero6, float* const* g1_5, float* const* g2_5, uint8_t* sh_packed,
                   float* sh_quant_bounds, uint8_t* sh_value_packed, float* sh_value_bounds, const NonShQuantState& non_sh, const float* radii,
                   const float* lrs, const float* reg, float sh_reg_weight, int step, const int32_t* steps) {
    typedef Vanilla3DGS<DEG> Prim;
    float* g1_6[6] = {g1_5[0], g1_5[1], g1_5[2], g1_5[3], g1_5[4], nullptr};
    float* g2_6[6] = {g2_5[0], g2_5[1], g2_5[2], g2_5[3], g2_5[4], nullptr};
    L1World<Prim> world(N, world6), v_world(N, zero6), g1(N, g1_6), g2(N, g2_6);
    L1Screen<Prim> v_screen((int64_t)C * N, v_screen5);
    fused_projection_bwd_optimizer_3dgs_kernel_wrapper<Prim, CameraModelType::PINHOLE, CameraDistortionType::None, AGNOSTIC, false, 1>(
        0, C, N, 15, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer((float*)nullptr), W, H,
        index, index + (N + 1), index + (N + 1) + (size_t)C * N, (const float4*)aabb, v_world, v_screen, g1, g2, sh_packed, (float4*)sh_quant_bounds,
        sh_value_packed, (float2*)sh_value_bounds, non_sh, radii, nullptr, lrs[0], lrs[1], lrs[2], lrs[3], lrs[4], lrs[5],
        reg[0], reg[1], reg[2], reg[3], reg[4], reg[5], reg[6], sh_reg_weight, 0.0f, step, steps);
}

extern "C" int ref_fpbo_l1(
    uint32_t C, uint32_t N, uint32_t W, uint32_t H, int sh_degree, float* const* world6, const float* viewmats, const float* intrins, const float* aabb,
    float* const* v_screen5, float* const* zero6, float* const* g1_5, float* const* g2_5, uint8_t* sh_packed, float* sh_quant_bounds,
    uint8_t* sh_value_packed, float* sh_value_bounds, uint8_t* const* nq_packed, float* const* nq_bounds, const float* radii, const float* lrs,
    const float* reg, float sh_reg_weight, int use_scale_agnostic_mean, int step, const int32_t* steps) {
    if (sh_degree != 3 && sh_degree != 1) return -1;
    NonShQuantState non_sh;
    if (nq_packed) {
        non_sh.enabled = true;
        non_sh.means_packed = nq_packed[0]; non_sh.quats_packed = nq_packed[1]; non_sh.scales_packed = nq_packed[2];
        non_sh.opacities_packed = nq_packed[3]; non_sh.features_dc_packed = nq_packed[4];
        non_sh.means_bounds = (float4*)nq_bounds[0]; non_sh.quats_bounds = (float4*)nq_bounds[1]; non_sh.scales_bounds = (float4*)nq_bounds[2];
        non_sh.opacities_bounds = (float4*)nq_bounds[3]; non_sh.features_dc_bounds = (float4*)nq_bounds[4];
    }
    std::vector<int32_t> h((size_t)N + 1 + 2 * (size_t)C * N);
    int32_t *bounds = h.data(), *cam = bounds + N + 1, *perm = cam + (size_t)C * N;
    for (uint32_t g = 0; g <= N; ++g) bounds[g] = (int32_t)(g * C);
    for (uint32_t c = 0; c < C; ++c)
        for (uint32_t g = 0; g < N; ++g) { cam[(size_t)c * N + g] = (int32_t)c; perm[(size_t)g * C + c] = (int32_t)(c * N + g); }
    int32_t* index = nullptr;
    if (cudaMalloc(&index, h.size() * sizeof(int32_t)) != cudaSuccess) return (int)cudaGetLastError();
    cudaMemcpy(index, h.data(), h.size() * sizeof(int32_t), cudaMemcpyHostToDevice);
#define RUN(DEG, AG) run_l1<DEG, AG>(C, N, W, H, world6, viewmats, intrins, index, aabb, v_screen5, zero6, g1_5, g2_5, sh_packed, sh_quant_bounds, \
                                    sh_value_packed, sh_value_bounds, non_sh, radii, lrs, reg, sh_reg_weight, step, steps)
    if (sh_degree == 3) { if (use_scale_agnostic_mean) RUN(3, true); else RUN(3, false); }
    else { if (use_scale_agnostic_mean) RUN(1, true); else RUN(1, false); }
#undef RUN
    const int rc = (int)cudaDeviceSynchronize();
    cudaFree(index);
    return rc;
}
