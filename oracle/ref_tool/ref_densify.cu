// TEST INFRASTRUCTURE.  The reference's densification kernels, compiled from where they lie
// (src/kernels/densify/*.cu with the Slang-generated device code the reference ships under src/generated/),
// behind plain-pointer entry points for the fixture generator and the live comparisons.
#include "kernels/densify/Quantile.cu"
#include "kernels/densify/DensifySampling.cu"
#include "kernels/densify/DensifyScoring.cu"
#include "kernels/densify/DensifySplitFilter.cu"
#include "kernels/densify/Relocation.cu"
#include "kernels/densify/McmcRelocation.cu"
#include "ref_sync.h"

template <class T>
static DeviceVector<T> vec_of(const void* p, int64_t n) {
    return DeviceVector<T>(TorchTensorView((uint64_t)p, 4, {n, (int64_t)(sizeof(T) / 4)}));
}

// densify_clip_scale_tensor (DensifyScoring.cu:180-197)
extern "C" int ref_densify_clip_scale(int64_t n, const float* radii, float* log_scales, float* logit_opacs, float max_scale2d, float hardness,
                                      float max_scale3d) {
    densify_clip_scale_tensor(n, vec_of<float>(radii, n), vec_of<float3>(log_scales, n), logit_opacs, max_scale2d, hardness, max_scale3d);
    return ref_finish();
}

// densify_accum_finalize_tensor (:296-304), densify_update_weight (:388-409), densify_clip_score_tensor (:346-385)
extern "C" int ref_densify_accum_finalize(int64_t n, float* accum) {
    densify_accum_finalize_tensor(n, vec_of<float>(accum, 2 * n));
    return ref_finish();
}

extern "C" int ref_densify_update_weight(int64_t n, const float* radii, const float* opacs, const float* score, const float* score2, float blend_w,
                                         float score_power, float* accum_buffer, int score_mode) {
    densify_update_weight(n, vec_of<float>(radii, n), nullptr, (float*)opacs, vec_of<float>(score, n),
                          score2 ? vec_of<float>(score2, n) : DeviceVector<float>(), blend_w, score_power, vec_of<float2>(accum_buffer, n), score_mode);
    return ref_finish();
}

extern "C" int ref_densify_clip_score(int64_t n, float* accum_buffer, float quantile, float power, float* score_out) {
    densify_clip_score_tensor(n, vec_of<float2>(accum_buffer, n), quantile, power, score_out ? vec_of<float2>(score_out, n) : DeviceVector<float2>());
    return ref_finish();
}

// mcmc_add_noise_tensor / revised_add_noise_tensor (McmcRelocation.cu:610-654)
extern "C" int ref_densify_add_noise(int64_t n, float scaler, int revised, const float* radii, float* means, const float* log_scales, const float* quats,
                                     const float* opacs) {
    if (revised)
        revised_add_noise_tensor(n, scaler, vec_of<float>(radii, n), vec_of<float3>(means, n), vec_of<float3>(log_scales, n), vec_of<float4>(quats, n),
                                 vec_of<float>(opacs, n));
    else
        mcmc_add_noise_tensor(n, scaler, vec_of<float3>(means, n), vec_of<float3>(log_scales, n), vec_of<float4>(quats, n), vec_of<float>(opacs, n));
    return ref_finish();
}

// relocate_splats_with_long_axis_split_tensor (mode 0) / add_splats_with_long_axis_split_tensor (mode 1), Relocation.cu:205-369.
// cap: allocated splats of every array; sh may be NULL (quantised values), the SH moments too (quantised state).
// Bounds are in the one-per-256-cells layout.  Non-SH moments stay fp32.
extern "C" int ref_densify_split(int mode, int64_t cur_n, int64_t num_new, int64_t cap, float min_opacity, float split_k, uint32_t seed,
                                 float* weights, float* means, float* quats, float* scales, float* opacs, float* dc, float* sh,
                                 float* m1_means, float* m1_quats, float* m1_scales, float* m1_opacs, float* m1_dc, float* m1_sh,
                                 float* m2_means, float* m2_quats, float* m2_scales, float* m2_opacs, float* m2_dc, float* m2_sh,
                                 uint8_t* sh_optim_packed, float* sh_optim_bounds, int sh_optim_bits, uint8_t* sh_value_packed, float* sh_value_bounds,
                                 int sh_value_bits, float* accum, int32_t* steps) {
    const int K = 15;
    const int64_t cells = cap * K * 3, blocks = (cells + 255) / 256;
    auto v3 = [&](float* p, int64_t n) { return p ? vec_of<float3>(p, n) : DeviceVector<float3>(); };
    DeviceVector<float3> g1sh, g2sh;
    if (sh_optim_bits == 32) { g1sh = v3(m1_sh, cap * K); g2sh = v3(m2_sh, cap * K); }
    else { g1sh = DeviceVector<float3>(TorchTensorView((uint64_t)sh_optim_packed, 1, {cap * K, 12LL})); g2sh = g1sh; }     // as engine_densify_step aliases them
    DeviceVector<float4> ob = sh_optim_bits == 32 ? DeviceVector<float4>() : vec_of<float4>(sh_optim_bounds, blocks);
    DeviceVector<uint8_t> vp = sh_value_bits == 32 ? DeviceVector<uint8_t>()
                                                   : DeviceVector<uint8_t>(TorchTensorView((uint64_t)sh_value_packed, 1, {cells * (sh_value_bits / 8)}));
    DeviceVector<float2> vb = sh_value_bits == 32 ? DeviceVector<float2>() : vec_of<float2>(sh_value_bounds, blocks);
    DeviceVector<int32_t> st = steps ? DeviceVector<int32_t>(TorchTensorView((uint64_t)steps, 4, {cap})) : DeviceVector<int32_t>();
    NonShQuantState non_sh{};
    if (mode == 0)
        relocate_splats_with_long_axis_split_tensor(cur_n, min_opacity, split_k, v3(means, cap), vec_of<float4>(quats, cap), v3(scales, cap),
            vec_of<float>(opacs, cap), v3(dc, cap), v3(sh, cap * K), v3(m1_means, cap), vec_of<float4>(m1_quats, cap), v3(m1_scales, cap),
            vec_of<float>(m1_opacs, cap), v3(m1_dc, cap), g1sh, v3(m2_means, cap), vec_of<float4>(m2_quats, cap), v3(m2_scales, cap),
            vec_of<float>(m2_opacs, cap), v3(m2_dc, cap), g2sh, vec_of<float2>(accum, cap), vec_of<float2>(weights, cap), st, sh_optim_bits, K, ob, false,
            vp, vb, sh_value_bits, false, K, non_sh, seed);
    else
        add_splats_with_long_axis_split_tensor(cur_n, num_new, split_k, v3(means, cap), vec_of<float4>(quats, cap), v3(scales, cap),
            vec_of<float>(opacs, cap), v3(dc, cap), v3(sh, cap * K), v3(m1_means, cap), vec_of<float4>(m1_quats, cap), v3(m1_scales, cap),
            vec_of<float>(m1_opacs, cap), v3(m1_dc, cap), g1sh, v3(m2_means, cap), vec_of<float4>(m2_quats, cap), v3(m2_scales, cap),
            vec_of<float>(m2_opacs, cap), v3(m2_dc, cap), g2sh, vec_of<float2>(accum, cap), vec_of<float2>(weights, cap), st, sh_optim_bits, K, ob, false,
            vp, vb, sh_value_bits, false, K, non_sh, seed);
    return ref_finish();
}
