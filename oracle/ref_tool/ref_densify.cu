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
