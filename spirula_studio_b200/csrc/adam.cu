// Adam updates for every Gaussian parameter, and the block-quantised codecs of
// the SH coefficients and their optimiser state.
//
// Restates fused_optim_3dgs_geometry_kernel (src/kernels/optim/FusedGeometryOptim.cu:83-380,
// fp32 moments; the regularisers, the scale-agnostic mean and per-splat steps in the EX
// instantiation), fused_adam_with_steps_kernel
// (src/kernels/optim/FusedAppearanceOptim.cu:11-56), fused_adam_with_steps_qq_kernel
// (:291-418) and the codecs QuantizedTensor / QuantizedAdamState
// (src/core/Tensor.h:978-1136,1313-1404).  beta1 = 0.9, beta2 = 0.999 and
// eps = 1e-15 added after the second moment is bias-corrected.
//
// All kernels are streaming: every byte is touched once, with 16-byte accesses
// where the layout allows it.
#include "ssb_common.cuh"

namespace ssb {

constexpr float kBeta1 = 0.9f, kBeta2 = 0.999f, kAdamEps = 1e-15f;

struct AdamScalars { float ibc1, ibc2; };

__device__ __forceinline__ float adam_update(float x, float g, float& m1, float& m2, float lr_ibc1, float ibc2) {
    m1 = kBeta1 * m1 + (1.f - kBeta1) * g;
    m2 = kBeta2 * m2 + (1.f - kBeta2) * g * g;
    return x - lr_ibc1 * m1 / (sqrtf(m2 * ibc2) + kAdamEps);
}

__device__ __forceinline__ float inv_bias_correction(float beta, float step) { return 1.0f / (1.0f - powf(beta, step)); }

// Peer mode (PEER = true) of the optimiser kernels: the gradient of a value is the sum of this rank's partial
// gradient and the partial gradients the other ranks hold at the same place of their own gradient buffers
// (read over NVLink, bypassing L1: a line cached by an earlier iteration would be stale), and an updated
// parameter is stored into every rank's replica.  Every buffer has the same layout on every rank, so another
// rank's copy of an address is that address plus a per-rank displacement.  Inbound gradient traffic and outbound
// parameter traffic of a CTA overlap, and the summed gradient never travels back to memory.
struct PeerOffsets {
    int32_t n;        // other ranks, 0..7
    int32_t pad;
    int64_t grads[SSB_MAX_PEERS - 1], params[SSB_MAX_PEERS - 1], sh_packed[SSB_MAX_PEERS - 1], sh_bounds[SSB_MAX_PEERS - 1];   // bytes
    // PEER == 2: displacement from this rank's copy to the buffer's NVSwitch multicast address, one address that reaches
    // every rank's copy: a load from it returns the switch's sum over all ranks (this one included), a store to it lands in
    // every replica.  Each rank then receives its range once instead of once per peer, and sends each update once.
    int64_t mc_grads, mc_params, mc_sh_packed, mc_sh_bounds;
};

__device__ __forceinline__ float4 multimem_sum4(const void* mc) {
    float4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc) : "memory");
    return r;
}
__device__ __forceinline__ float multimem_sum1(const void* mc) {
    float r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(r) : "l"(mc) : "memory");
    return r;
}
__device__ __forceinline__ void multimem_store(void* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}
__device__ __forceinline__ void multimem_store(void* mc, const uint2& v) {
    asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" :: "l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)) : "memory");
}
__device__ __forceinline__ void multimem_store(void* mc, uint32_t v) {
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" :: "l"(mc), "f"(__uint_as_float(v)) : "memory");
}

// 16-byte load that bypasses L1, as a volatile statement: a thread's loads from all ranks are issued back to back, in
// program order, before the first sum needs one of them.
__device__ __forceinline__ float4 ld_cv4(const void* p) {
    float4 r;
    asm volatile("ld.global.cv.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p));
    return r;
}

template <int PEER>
__device__ __forceinline__ float grad_sum(const float* own, const PeerOffsets& po) {
    if constexpr (PEER == 2) return multimem_sum1((const char*)own + po.mc_grads);
    float v = *own;
    if (PEER) {
        float x[SSB_MAX_PEERS - 1];
#pragma unroll
        for (int k = 0; k < SSB_MAX_PEERS - 1; ++k) x[k] = k < po.n ? __ldcv((const float*)((const char*)own + po.grads[k])) : 0.f;   // all in flight together
#pragma unroll
        for (int k = 0; k < SSB_MAX_PEERS - 1; ++k) v += x[k];
    }
    return v;
}
template <int PEER>
__device__ __forceinline__ float4 grad_sum4(const float4* own, const PeerOffsets& po) {
    if constexpr (!PEER) {
        return *own;
    } else if constexpr (PEER == 2) {
        return multimem_sum4((const char*)own + po.mc_grads);
    } else {
        float4 x[SSB_MAX_PEERS - 1];
#pragma unroll
        for (int k = 0; k < SSB_MAX_PEERS - 1; ++k) x[k] = ld_cv4((const char*)own + (k < po.n ? po.grads[k] : 0));   // unused slots re-read the own copy
        float4 v = *own;
#pragma unroll
        for (int k = 0; k < SSB_MAX_PEERS - 1; ++k)
            if (k < po.n) { v.x += x[k].x; v.y += x[k].y; v.z += x[k].z; v.w += x[k].w; }
        return v;
    }
}
// dst[0..count) (shared memory) = this rank's own[0..count) + every other rank's, 16 bytes per thread per step, the loads
// of all ranks in flight together; `own` must be 16-byte aligned.  Whole CTA; the caller synchronises afterwards.
template <int THREADS, int PEER>
__device__ __forceinline__ void peer_sum_to_shared(float* dst, const float* own, int count, const PeerOffsets& po) {
    const int n_vec = count >> 2;
    if constexpr (PEER == 2) {
        for (int v = threadIdx.x; v < n_vec; v += THREADS) ((float4*)dst)[v] = multimem_sum4((const char*)((const float4*)own + v) + po.mc_grads);
        for (int i = (n_vec << 2) + threadIdx.x; i < count; i += THREADS) dst[i] = multimem_sum1((const char*)(own + i) + po.mc_grads);
    } else {
        for (int v = threadIdx.x; v < n_vec; v += THREADS) {
            const char* at = (const char*)((const float4*)own + v);
            float4 x[SSB_MAX_PEERS - 1];
#pragma unroll
            for (int k = 0; k < SSB_MAX_PEERS - 1; ++k) x[k] = ld_cv4(at + (k < po.n ? po.grads[k] : 0));   // unused slots re-read the own copy
            float4 acc = *(const float4*)at;
#pragma unroll
            for (int k = 0; k < SSB_MAX_PEERS - 1; ++k)
                if (k < po.n) { acc.x += x[k].x; acc.y += x[k].y; acc.z += x[k].z; acc.w += x[k].w; }
            ((float4*)dst)[v] = acc;
        }
        for (int i = (n_vec << 2) + threadIdx.x; i < count; i += THREADS) {
            float acc = own[i];
            for (int k = 0; k < po.n; ++k) acc += __ldcv((const float*)((const char*)(own + i) + po.grads[k]));
            dst[i] = acc;
        }
    }
}

// own[0..count) and every other rank's copy of it = src[0..count) (shared memory), 16-byte stores.
template <int THREADS, int PEER>
__device__ __forceinline__ void shared_to_all(float* own, const float* src, int count, const PeerOffsets& po) {
    const int n_vec = count >> 2;
    if constexpr (PEER == 2) {
        for (int v = threadIdx.x; v < n_vec; v += THREADS) multimem_store((char*)((float4*)own + v) + po.mc_params, ((const uint4*)src)[v]);
        for (int i = (n_vec << 2) + threadIdx.x; i < count; i += THREADS) multimem_store((char*)(own + i) + po.mc_params, __float_as_uint(src[i]));
    } else {
        for (int v = threadIdx.x; v < n_vec; v += THREADS) {
            const float4 x = ((const float4*)src)[v];
            char* at = (char*)((float4*)own + v);
            *(float4*)at = x;
#pragma unroll
            for (int k = 0; k < SSB_MAX_PEERS - 1; ++k)
                if (k < po.n) *(float4*)(at + po.params[k]) = x;
        }
        for (int i = (n_vec << 2) + threadIdx.x; i < count; i += THREADS) {
            own[i] = src[i];
            for (int k = 0; k < po.n; ++k) *(float*)((char*)(own + i) + po.params[k]) = src[i];
        }
    }
}

// own copy and, in peer mode, every other rank's copy
template <int PEER, class T>
__device__ __forceinline__ void store_all(T* own, const T& v, const PeerOffsets& po, const int64_t (&disp)[SSB_MAX_PEERS - 1], int64_t mc_disp = 0) {
    if constexpr (PEER == 2 && (sizeof(T) == 16 || sizeof(T) == 8 || sizeof(T) == 4)) {
        // one store through the switch reaches every replica, this rank's included
        if constexpr (sizeof(T) == 16) multimem_store((char*)own + mc_disp, *(const uint4*)&v);
        else if constexpr (sizeof(T) == 8) multimem_store((char*)own + mc_disp, *(const uint2*)&v);
        else multimem_store((char*)own + mc_disp, *(const uint32_t*)&v);
        return;
    }
    *own = v;
    if (PEER) {
#pragma unroll
        for (int k = 0; k < SSB_MAX_PEERS - 1; ++k)
            if (k < po.n) *(T*)((char*)own + disp[k]) = v;
    }
}

// Gradients of the five per-splat regularisers with all loss cotangents 1 (reverse mode of
// per_splat_losses, src/shaders/per_splat_losses.slang:5-141) for log-scales s, logit opacity o and
// the normalised quaternion q.  The weights arrive divided by the splat count.
__device__ __forceinline__ void per_splat_reg_grads(const float s[3], float o, const float q[4], const SsbAdamExtras& ex, float inv_n,
                                                    float gs_out[3], float& go_out, float gq_out[4]) {
    // mcmc opacity: w * sigmoid(o)
    const float sg = 1.0f / (1.0f + expf(-o));
    go_out = ex.mcmc_opacity_reg_weight * inv_n * sg * (1.0f - sg);
    // mcmc scale: w * 1e-2 * (s0 + s1 + s2) / 3
    const float gm = ex.mcmc_scale_reg_weight * inv_n * 1e-2f / 3.0f;
    gs_out[0] = gs_out[1] = gs_out[2] = gm;
    // index of the largest and the smallest scale, ties broken as nested max(max(x, y), z) differentiates
    int imax = s[0] > s[1] ? 0 : 1; imax = s[imax] > s[2] ? imax : 2;
    int imin = s[0] < s[1] ? 0 : 1; imin = s[imin] < s[2] ? imin : 2;
    // scale ratio: w * (max(e_max / e_min, R) - R)
    {
        const float ratio = expf(s[imax]) / expf(s[imin]);
        if (ratio > ex.max_gauss_ratio) {
            const float w = ex.scale_regularization_weight * inv_n * ratio;
#pragma unroll
            for (int k = 0; k < 3; ++k) gs_out[k] += (k == imax ? w : 0.f) - (k == imin ? w : 0.f);
        }
    }
    // effective rank: E = exp(2 s), p1 = E_max / S, p3 = E_min / S, p2 = 1 - p1 - p3, r = exp(entropy(p));
    // loss = w * max(-log(r - 0.99999), 0) + w3 * p3
    {
        float E[3] = {expf(2.0f * s[0]), expf(2.0f * s[1]), expf(2.0f * s[2])};
        const float S = E[0] + E[1] + E[2];
        const float p1 = E[imax] / S, p3 = E[imin] / S, p2 = 1.0f - p1 - p3;
        const float l1 = logf(p1), l2 = logf(p2), l3 = logf(p3);
        const float r = expf(-p1 * l1 - p2 * l2 - p3 * l3);
        float dH = 0.f;
        if (-logf(r - 0.99999f) > 0.0f) dH = -ex.erank_reg_weight * inv_n / (r - 0.99999f) * r;
        const float dp1 = dH * (l2 - l1), dp3 = dH * (l2 - l3) + ex.erank_reg_weight_s3 * inv_n;
        const float dS = -(dp1 * p1 + dp3 * p3) / S;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            float dE = dS + (k == imax ? dp1 / S : 0.f) + (k == imin ? dp3 / S : 0.f);
            gs_out[k] += dE * 2.0f * E[k];
        }
    }
    // quaternion norm: w * (n - 1 - log n), n = |q|
    {
        const float n = sqrtf(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
        const float w = ex.quat_norm_reg_weight * inv_n * (1.0f - 1.0f / n) / n;
#pragma unroll
        for (int k = 0; k < 4; ++k) gq_out[k] = w * q[k];
    }
}

// Order-preserving map float -> uint32, so min/max run on the integer redux unit.
__device__ __forceinline__ uint32_t f2ord(float f) {
    uint32_t b = __float_as_uint(f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}
__device__ __forceinline__ float ord2f(uint32_t k) {
    return __uint_as_float(k ^ ((k >> 31) ? 0x80000000u : 0xffffffffu));
}

// Block-wide (256 threads) minima of NMIN values and maxima of NMAX values in two barriers:
// one redux.sync per value in each warp, 8 partials per value through shared memory, then
// one more redux by the first warp.
template <int NMIN, int NMAX>
__device__ __forceinline__ void block_minmax(const float (&vmin)[NMIN], const float (&vmax)[NMAX], float (&omin)[NMIN], float (&omax)[NMAX],
                                             uint32_t (*sh)[8]) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t r[NMIN + NMAX];
#pragma unroll
    for (int k = 0; k < NMIN; ++k) r[k] = __reduce_min_sync(0xffffffffu, f2ord(vmin[k]));
#pragma unroll
    for (int k = 0; k < NMAX; ++k) r[NMIN + k] = __reduce_max_sync(0xffffffffu, f2ord(vmax[k]));
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < NMIN + NMAX; ++k) sh[k][w] = r[k];
    }
    __syncthreads();
    if (w == 0) {
#pragma unroll
        for (int k = 0; k < NMIN + NMAX; ++k) {
            uint32_t v = sh[k][lane & 7];
            v = k < NMIN ? __reduce_min_sync(0xffffffffu, v) : __reduce_max_sync(0xffffffffu, v);
            if (lane == 0) sh[k][0] = v;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NMIN; ++k) omin[k] = ord2f(sh[k][0]);
#pragma unroll
    for (int k = 0; k < NMAX; ++k) omax[k] = ord2f(sh[NMIN + k][0]);
}

// geometry (means, quats, scales, opacities) + features_dc, one thread per splat.
// EX adds the per-splat regularisers, the scale-agnostic mean update and per-splat step counters.
// NQ: the moments of the five arrays live in 16-bit joint codes (u = g1 / (sqrt(g2) + eps), log1p(sqrt(g2) / eps)), four bytes per
// cell, with one float4 of bounds per 256 splats and array (QuantizedAdamState<16, 256>, src/core/Tensor.h:978-1136; the
// non_sh_quant path of fused_optim_3dgs_geometry_kernel, src/kernels/optim/FusedGeometryOptim.cu:144-380).  A CTA is one block
// of 256 splats: every thread decodes its splat's 14 moment pairs into shared memory, the update below runs on them unchanged,
// then the block's new bounds are reduced and the pairs encoded again.
struct MomentsQ16 { uint8_t* packed[5]; float4* bounds[5]; };   // means, quats, scales, opacities, features_dc

__device__ __forceinline__ void q16_decode(const uint8_t* packed, int64_t cell, float4 mm, float& g1, float& g2) {
    const uint32_t w = ((const uint32_t*)packed)[cell];
    const float u = mm.x + (mm.y - mm.x) * ((float)(w & 0xffffu) * (1.0f / 65535.0f));
    const float ls = mm.z + (mm.w - mm.z) * ((float)(w >> 16) * (1.0f / 65535.0f));
    const float sq = kAdamEps * expm1f(ls);
    g1 = u * (sq + kAdamEps);
    g2 = sq * sq;
}
__device__ __forceinline__ void q16_us(float g1, float g2, float& u, float& ls) {
    const float sq = sqrtf(fmaxf(g2, 0.0f));
    u = g1 / (sq + kAdamEps);
    ls = log1pf(sq * (1.0f / kAdamEps));
}
__device__ __forceinline__ uint32_t q16_encode(float u, float ls, float4 mm) {
    const float ur = fmaxf(mm.y - mm.x, kAdamEps), sr = fmaxf(mm.w - mm.z, kAdamEps);
    const float uq = fminf(fmaxf(roundf(65535.0f * (u - mm.x) / ur), 0.0f), 65535.0f);
    const float sq = fminf(fmaxf(roundf(65535.0f * (ls - mm.z) / sr), 0.0f), 65535.0f);
    return (uint32_t)uq | ((uint32_t)sq << 16);
}

template <bool EX, int PEER, bool NQ = false>
__global__ void __launch_bounds__(256) adam_geometry_kernel(
    SsbSplats p, SsbSplats g, SsbSplats m1, SsbSplats m2, int64_t first, int64_t count, SsbAdamConfig cfg,
    float ibc1, float ibc2, float dc_decay, SsbAdamExtras ex, PeerOffsets po, MomentsQ16 nq = MomentsQ16{}) {
    int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    static_assert(!(NQ && PEER == 2), "the quantised moments take per-peer loads and stores, not the multicast address");
    constexpr int kMom = NQ ? 14 * 256 : 4;
    __shared__ __align__(16) float mom1[kMom], mom2[kMom];
    __shared__ uint32_t mm_sh[NQ ? 20 : 1][8];
    if constexpr (NQ) {
        // layout per array as in global memory, indexed with the splat's own number through moved-back pointers
        const int64_t blk0 = first + (int64_t)blockIdx.x * 256;
        float* a = mom1; float* b = mom2;
        m1.means = a - 3 * blk0; m1.quats = a + 768 - 4 * blk0; m1.scales = a + 1792 - 3 * blk0; m1.opacities = a + 2560 - blk0; m1.features_dc = a + 2816 - 3 * blk0;
        m2.means = b - 3 * blk0; m2.quats = b + 768 - 4 * blk0; m2.scales = b + 1792 - 3 * blk0; m2.opacities = b + 2560 - blk0; m2.features_dc = b + 2816 - 3 * blk0;
        if (i < first + count) {
            const int64_t blk = i >> 8;
            const int width[5] = {3, 4, 3, 1, 3};
            float* d1[5] = {m1.means, m1.quats, m1.scales, m1.opacities, m1.features_dc};
            float* d2[5] = {m2.means, m2.quats, m2.scales, m2.opacities, m2.features_dc};
#pragma unroll
            for (int t = 0; t < 5; ++t) {
                const float4 mm = nq.bounds[t][blk];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (k < width[t]) q16_decode(nq.packed[t], (int64_t)width[t] * i + k, mm, d1[t][(int64_t)width[t] * i + k], d2[t][(int64_t)width[t] * i + k]);
            }
        }
    }
    // Peer mode: the CTA's 256 splats are contiguous in each array, so their gradients are summed over the ranks
    // with coalesced 16-byte loads into shared memory, each thread then works from there, leaves its updated
    // parameters in the same place, and the CTA stores them into every replica with 16-byte stores.
    constexpr int kStage = PEER ? 14 * 256 : 4;
    __shared__ __align__(16) float stage[kStage];
    const int64_t b0 = first + (int64_t)blockIdx.x * 256;
    const int nb = (int)min((int64_t)256, first + count - b0);
    SsbSplats g_own = g;                 // where zeroing goes
    SsbSplats out = p;                   // where updated parameters go
    if constexpr (PEER) {
        float* s_means = stage, *s_quats = stage + 768, *s_scales = stage + 1792, *s_opac = stage + 2560, *s_dc = stage + 2816;
        peer_sum_to_shared<256, PEER>(s_means, g.means + 3 * b0, 3 * nb, po);
        peer_sum_to_shared<256, PEER>(s_quats, g.quats + 4 * b0, 4 * nb, po);
        peer_sum_to_shared<256, PEER>(s_scales, g.scales + 3 * b0, 3 * nb, po);
        peer_sum_to_shared<256, PEER>(s_opac, g.opacities + b0, nb, po);
        peer_sum_to_shared<256, PEER>(s_dc, g.features_dc + 3 * b0, 3 * nb, po);
        __syncthreads();
        // indexed with the global splat index like the arrays they stand in for
        g.means = s_means - 3 * b0; g.quats = s_quats - 4 * b0; g.scales = s_scales - 3 * b0; g.opacities = s_opac - b0; g.features_dc = s_dc - 3 * b0;
        out = g;
    }
    if (i < first + count) {
    const float gs = cfg.grad_scale;
    const bool zg = cfg.zero_grad != 0;
    float reg_s[3] = {0.f, 0.f, 0.f}, reg_o = 0.f, reg_q[4] = {0.f, 0.f, 0.f, 0.f};
    float s_old[3] = {0.f, 0.f, 0.f}, o_old = 0.f, qn_old[4] = {1.f, 0.f, 0.f, 0.f};
    if (EX) {
        if (ex.d_steps) {
            const float step = (float)ex.d_steps[i];
            ibc1 = inv_bias_correction(kBeta1, step);
            ibc2 = inv_bias_correction(kBeta2, step);
        }
        const float4 q4 = ((const float4*)p.quats)[i];
        const float inv = 1.0f / sqrtf(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w);
        qn_old[0] = q4.x * inv; qn_old[1] = q4.y * inv; qn_old[2] = q4.z * inv; qn_old[3] = q4.w * inv;
#pragma unroll
        for (int k = 0; k < 3; ++k) s_old[k] = p.scales[3 * i + k];
        o_old = p.opacities[i];
        per_splat_reg_grads(s_old, o_old, qn_old, ex, 1.0f / (float)ex.n_total, reg_s, reg_o, reg_q);
    }
    const float lr_s = cfg.lr_scales * ibc1, lr_q = cfg.lr_quats * ibc1, lr_o = cfg.lr_opacities * ibc1, lr_m = cfg.lr_means * ibc1;
    const float lr_dc = cfg.lr_features_dc * ibc1;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        int64_t q = 3 * i + k;
        float a = m1.scales[q], b = m2.scales[q];
        out.scales[q] = adam_update(p.scales[q], reg_s[k] + gs * g.scales[q], a, b, lr_s, ibc2);
        m1.scales[q] = a; m2.scales[q] = b;
        if (zg) g_own.scales[q] = 0.f;
    }
    {
        float4 q4 = ((float4*)p.quats)[i], g4 = ((float4*)g.quats)[i];
        float4 a4 = ((float4*)m1.quats)[i], b4 = ((float4*)m2.quats)[i];
        float inv = 1.0f / sqrtf(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w);
        float q[4] = {q4.x * inv, q4.y * inv, q4.z * inv, q4.w * inv};
        float gq[4] = {reg_q[0] + gs * g4.x, reg_q[1] + gs * g4.y, reg_q[2] + gs * g4.z, reg_q[3] + gs * g4.w};
        float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
        float dq = q[0] * gq[0] + q[1] * gq[1] + q[2] * gq[2] + q[3] * gq[3];
        float u[4], n2 = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float gk = gq[k] - dq * q[k];
            u[k] = adam_update(q[k], gk, a[k], b[k], lr_q, ibc2);
            n2 += u[k] * u[k];
        }
        float inv2 = 1.0f / sqrtf(n2);
        ((float4*)out.quats)[i] = make_float4(u[0] * inv2, u[1] * inv2, u[2] * inv2, u[3] * inv2);
        ((float4*)m1.quats)[i] = make_float4(a[0], a[1], a[2], a[3]);
        ((float4*)m2.quats)[i] = make_float4(b[0], b[1], b[2], b[3]);
        if (zg) ((float4*)g_own.quats)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    {
        float a = m1.opacities[i], b = m2.opacities[i];
        out.opacities[i] = adam_update(p.opacities[i], reg_o + gs * g.opacities[i], a, b, lr_o, ibc2);
        m1.opacities[i] = a; m2.opacities[i] = b;
        if (zg) g_own.opacities[i] = 0.f;
    }
    const float gm[3] = {g.means[3 * i], g.means[3 * i + 1], g.means[3 * i + 2]};
    if (EX && ex.d_densify_score) {
        const float vx = gs * gm[0], vy = gs * gm[1], vz = gs * gm[2];
        ex.d_densify_score[i] = expf(fmaxf(fmaxf(s_old[0], s_old[1]), s_old[2])) * sqrtf(vx * vx + vy * vy + vz * vz);
    }
    if (EX && ex.use_scale_agnostic_mean) {
        // first moment of covariance * gradient * sqrt(2 log(255 * opacity)), second moment of
        // (gradient * 0.6 * screen radius)^2, all from the parameters before this update
        float v[3] = {gs * gm[0], gs * gm[1], gs * gm[2]};
        const float w = qn_old[0], x = qn_old[1], y = qn_old[2], z = qn_old[3];
        const float R[9] = {1.f - 2.f * (y * y + z * z), 2.f * (x * y - w * z), 2.f * (x * z + w * y),
                            2.f * (x * y + w * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z - w * x),
                            2.f * (x * z - w * y), 2.f * (y * z + w * x), 1.f - 2.f * (x * x + y * y)};
        float t[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) t[k] = expf(s_old[k]) * (R[k] * v[0] + R[3 + k] * v[1] + R[6 + k] * v[2]);   // S^2 R^T v
        const float sg = 1.0f / (1.0f + expf(-o_old));
        const float ext = sqrtf(2.0f * logf(fmaxf(255.0f * sg, 1.00001f)));
        const float den = ex.d_radii[i] * 0.6f;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            int64_t q = 3 * i + k;
            const float num = (R[3 * k] * t[0] + R[3 * k + 1] * t[1] + R[3 * k + 2] * t[2]) * ext;
            float a = m1.means[q], b = m2.means[q];
            a = kBeta1 * a + (1.f - kBeta1) * num;
            b = kBeta2 * b + (1.f - kBeta2) * v[k] * v[k] * den * den;
            out.means[q] = p.means[q] - lr_m * a / (sqrtf(b * ibc2) + kAdamEps);
            m1.means[q] = a; m2.means[q] = b;
            if (zg) g_own.means[q] = 0.f;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            int64_t q = 3 * i + k;
            float a = m1.means[q], b = m2.means[q];
            out.means[q] = adam_update(p.means[q], gs * gm[k], a, b, lr_m, ibc2);
            m1.means[q] = a; m2.means[q] = b;
            if (zg) g_own.means[q] = 0.f;
        }
    }
    const float dc_off = 0.5f / 0.28209479177387814f;
    if (p.features_dc)        // NULL: the caller updates DC with the plain kernel, as the reference's fp32 path does
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        int64_t q = 3 * i + k;
        float x = p.features_dc[q], v = g.features_dc[q];
        if (!isfinite(v)) v = 0.f;
        v *= gs;
        v += dc_decay * (fmaxf(x - dc_off, 0.0f) + fminf(x + dc_off, 0.0f));
        float a = m1.features_dc[q], b = m2.features_dc[q];
        out.features_dc[q] = adam_update(x, v, a, b, lr_dc, ibc2);
        m1.features_dc[q] = a; m2.features_dc[q] = b;
        if (zg) g_own.features_dc[q] = 0.f;
    }
    }   // this thread's splat
    if constexpr (NQ) {
        // new bounds of the block (u and log-s ranges per array), then the codes
        const bool inside = i < first + count;
        const int width[5] = {3, 4, 3, 1, 3};
        float* d1[5] = {m1.means, m1.quats, m1.scales, m1.opacities, m1.features_dc};
        float* d2[5] = {m2.means, m2.quats, m2.scales, m2.opacities, m2.features_dc};
        float u[14], ls[14], mn[10], mx[10];
        int c = 0;
#pragma unroll
        for (int t = 0; t < 5; ++t) {
            mn[2 * t] = mn[2 * t + 1] = 1e30f; mx[2 * t] = mx[2 * t + 1] = -1e30f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (k < width[t]) {
                    u[c] = ls[c] = 0.f;
                    if (inside) {
                        q16_us(d1[t][(int64_t)width[t] * i + k], d2[t][(int64_t)width[t] * i + k], u[c], ls[c]);
                        mn[2 * t] = fminf(mn[2 * t], u[c]); mx[2 * t] = fmaxf(mx[2 * t], u[c]);
                        mn[2 * t + 1] = fminf(mn[2 * t + 1], ls[c]); mx[2 * t + 1] = fmaxf(mx[2 * t + 1], ls[c]);
                    }
                    ++c;
                }
        }
        float omn[10], omx[10];
        block_minmax<10, 10>(mn, mx, omn, omx, mm_sh);
        const int64_t blk = (first + (int64_t)blockIdx.x * 256) >> 8;
        c = 0;
#pragma unroll
        for (int t = 0; t < 5; ++t) {
            const float4 mm = make_float4(omn[2 * t], omx[2 * t], omn[2 * t + 1], omx[2 * t + 1]);
            if (threadIdx.x == 0) nq.bounds[t][blk] = mm;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (k < width[t]) {
                    if (inside) ((uint32_t*)nq.packed[t])[(int64_t)width[t] * i + k] = q16_encode(u[c], ls[c], mm);
                    ++c;
                }
        }
    }
    if constexpr (PEER) {
        __syncthreads();
        shared_to_all<256, PEER>(p.means + 3 * b0, stage, 3 * nb, po);
        shared_to_all<256, PEER>(p.quats + 4 * b0, stage + 768, 4 * nb, po);
        shared_to_all<256, PEER>(p.scales + 3 * b0, stage + 1792, 3 * nb, po);
        shared_to_all<256, PEER>(p.opacities + b0, stage + 2560, nb, po);
        shared_to_all<256, PEER>(p.features_dc + 3 * b0, stage + 2816, 3 * nb, po);
    }
}

// element-wise Adam (features_sh), four floats per thread
template <int PEER>
__global__ void __launch_bounds__(256) adam_plain_kernel(
    float* __restrict__ param, float* __restrict__ grad, float* __restrict__ m1, float* __restrict__ m2, int64_t numel,
    float lr_ibc1, float ibc2, float decay, float decay_offset, float grad_scale, int zero_grad,
    const int32_t* __restrict__ steps, int stride, float lr, PeerOffsets po) {
    int64_t i4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i4 >= numel) return;
    if (steps) {
        // per-splat step counters: element i uses steps[i / stride]; `steps` is already offset to the range's first splat
        for (int64_t i = i4; i < numel && i < i4 + 4; ++i) {
            const float step = (float)steps[i / stride];
            float x = param[i], gk = grad_sum<PEER>(grad + i, po);
            if (!isfinite(gk)) gk = 0.f;
            gk *= grad_scale;
            gk += decay * (fmaxf(x - decay_offset, 0.0f) + fminf(x + decay_offset, 0.0f));
            float a = m1[i], b = m2[i];
            store_all<PEER>(param + i, adam_update(x, gk, a, b, lr * inv_bias_correction(kBeta1, step), inv_bias_correction(kBeta2, step)), po, po.params, po.mc_params);
            m1[i] = a; m2[i] = b;
            if (zero_grad) grad[i] = 0.f;
        }
        return;
    }
    if (i4 + 4 <= numel && ((((uintptr_t)param | (uintptr_t)grad | (uintptr_t)m1 | (uintptr_t)m2) & 15) == 0)) {
        float4 x = *(float4*)(param + i4), v = grad_sum4<PEER>((const float4*)(grad + i4), po), a = *(float4*)(m1 + i4), b = *(float4*)(m2 + i4);
        float xs[4] = {x.x, x.y, x.z, x.w}, vs[4] = {v.x, v.y, v.z, v.w}, as[4] = {a.x, a.y, a.z, a.w}, bs[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float gk = isfinite(vs[k]) ? vs[k] : 0.f;
            gk *= grad_scale;
            gk += decay * (fmaxf(xs[k] - decay_offset, 0.0f) + fminf(xs[k] + decay_offset, 0.0f));
            xs[k] = adam_update(xs[k], gk, as[k], bs[k], lr_ibc1, ibc2);
        }
        store_all<PEER>((float4*)(param + i4), make_float4(xs[0], xs[1], xs[2], xs[3]), po, po.params, po.mc_params);
        *(float4*)(m1 + i4) = make_float4(as[0], as[1], as[2], as[3]);
        *(float4*)(m2 + i4) = make_float4(bs[0], bs[1], bs[2], bs[3]);
        if (zero_grad) *(float4*)(grad + i4) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        for (int64_t i = i4; i < numel && i < i4 + 4; ++i) {
            float x = param[i], gk = grad_sum<PEER>(grad + i, po);
            if (!isfinite(gk)) gk = 0.f;
            gk *= grad_scale;
            gk += decay * (fmaxf(x - decay_offset, 0.0f) + fminf(x + decay_offset, 0.0f));
            float a = m1[i], b = m2[i];
            store_all<PEER>(param + i, adam_update(x, gk, a, b, lr_ibc1, ibc2), po, po.params, po.mc_params);
            m1[i] = a; m2[i] = b;
            if (zero_grad) grad[i] = 0.f;
        }
    }
}

__device__ __forceinline__ float sqrt_approx(float x) {
    float r;
    asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// One CTA of 64 threads = one 256-cell quantisation block, four consecutive cells per thread
// (16-byte gradient loads, 8-byte code loads); the block minima/maxima are folded per thread
// first, then one redux.sync per value per warp and a two-entry exchange through shared memory.
// OPTIM_BITS = 8: two bytes per cell (u, s); 4: one byte per cell, u in the low nibble (QuantizedAdamState<4,256>).
// STEPS: per-splat step counters (compiled apart: the power function costs the plain path registers).
// PEER: gradients summed over the ranks, value codes and value bounds stored into every replica (the values must then be
// packed, or, when plain fp32, part of the parameter buffer: their displacements are taken accordingly).
template <int VALUE_BITS, int OPTIM_BITS, bool STEPS, int PEER>
__global__ void __launch_bounds__(64) adam_qq_kernel(
    float* __restrict__ grad, uint8_t* __restrict__ optim_packed, float4* __restrict__ optim_bounds,
    uint8_t* __restrict__ value_packed, float2* __restrict__ value_bounds, int64_t first_block, int64_t numel_total,
    float lr_ibc1, float ibc2, float decay, float decay_offset, float grad_scale, int zero_grad,
    const int32_t* __restrict__ steps, int stride, float lr, PeerOffsets po) {
    __shared__ uint32_t sh[6][2];
    const int64_t blk = first_block + blockIdx.x;
    const int64_t idx0 = blk * 256 + threadIdx.x * 4;
    // VALUE_BITS == 32: the values are plain fp32 (only the optimiser state is quantised,
    // fused_adam_step_quantized, src/kernels/optim/FusedAppearanceOptim.cu:137-271)
    constexpr bool kPlainValue = VALUE_BITS == 32;
    constexpr float vq = kPlainValue ? 1.0f : (float)((1u << (VALUE_BITS & 31)) - 1u), vinv = 1.0f / vq;
    constexpr bool kNibbles = OPTIM_BITS == 4;
    const float oq = kNibbles ? 15.0f : 255.0f, oinv = 1.0f / oq;
    const float2 vmm = kPlainValue ? make_float2(0.f, 0.f) : value_bounds[blk];
    const float4 omm = optim_bounds[blk];
    float x[4], u_new[4], s_new[4];
    bool inside[4];
    float gv[4];
    uint32_t vcode[4], ucode[4], scode[4];
    const bool full = idx0 + 4 <= numel_total;
    [[maybe_unused]] int64_t step_splat = -1;
    [[maybe_unused]] float step_lr1 = 0.f, step_c2 = 0.f;
    if (full) {
        const float4 g4 = grad_sum4<PEER>((const float4*)(grad + idx0), po);
        gv[0] = g4.x; gv[1] = g4.y; gv[2] = g4.z; gv[3] = g4.w;
        if (kPlainValue) {
            const uint4 c = *(const uint4*)((const float*)value_packed + idx0);
            vcode[0] = c.x; vcode[1] = c.y; vcode[2] = c.z; vcode[3] = c.w;      // raw fp32 bits
        } else if (VALUE_BITS == 16) {
            const ushort4 c = *(const ushort4*)((const uint16_t*)value_packed + idx0);
            vcode[0] = c.x; vcode[1] = c.y; vcode[2] = c.z; vcode[3] = c.w;
        } else {
            const uchar4 c = *(const uchar4*)(value_packed + idx0);
            vcode[0] = c.x; vcode[1] = c.y; vcode[2] = c.z; vcode[3] = c.w;
        }
        if (kNibbles) {
            const uint32_t oc = *(const uint32_t*)(optim_packed + idx0);
#pragma unroll
            for (int k = 0; k < 4; ++k) { ucode[k] = (oc >> (8 * k)) & 15u; scode[k] = (oc >> (8 * k + 4)) & 15u; }
        } else {
            const uint2 oc = *(const uint2*)(optim_packed + 2 * idx0);
            ucode[0] = oc.x & 255u; scode[0] = (oc.x >> 8) & 255u; ucode[1] = (oc.x >> 16) & 255u; scode[1] = oc.x >> 24;
            ucode[2] = oc.y & 255u; scode[2] = (oc.y >> 8) & 255u; ucode[3] = (oc.y >> 16) & 255u; scode[3] = oc.y >> 24;
        }
        if (zero_grad) *(float4*)(grad + idx0) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int64_t idx = idx0 + k;
        inside[k] = idx < numel_total;
        if (!full && inside[k]) {
            gv[k] = grad_sum<PEER>(grad + idx, po);
            vcode[k] = kPlainValue ? ((const uint32_t*)value_packed)[idx]
                                   : VALUE_BITS == 8 ? (uint32_t)value_packed[idx] : (uint32_t)((const uint16_t*)value_packed)[idx];
            if (kNibbles) { const uint32_t b = optim_packed[idx]; ucode[k] = b & 15u; scode[k] = b >> 4; }
            else { ucode[k] = optim_packed[2 * idx]; scode[k] = optim_packed[2 * idx + 1]; }
            if (zero_grad) grad[idx] = 0.f;
        }
        x[k] = u_new[k] = s_new[k] = 0.f;
        if (inside[k]) {
            float xv = kPlainValue ? __uint_as_float(vcode[k]) : vmm.x + (vmm.y - vmm.x) * ((float)vcode[k] * vinv);
            float v = gv[k];
            if (!isfinite(v)) v = 0.f;
            v *= grad_scale;
            v += decay * (fmaxf(xv - decay_offset, 0.0f) + fminf(xv + decay_offset, 0.0f));
            float u = omm.x + (omm.y - omm.x) * ((float)ucode[k] * oinv);
            float ls = omm.z + (omm.w - omm.z) * ((float)scode[k] * oinv);
            // sqrt(g2) = eps * expm1(ls).  ls is either 0 (never-updated cell) or far above 1 (sqrt(g2)/eps is astronomically
            // large for any real gradient).  exp - 1 is exact at 0 (2^0 = 1) and expm1 to working precision above 1; in the band
            // between (a second moment below 1e-29, which no real gradient leaves behind) it loses digits nothing downstream sees.
            // A branch to the careful routine made every warp holding one never-updated cell run both.
            const float em1 = __expf(ls) - 1.0f;
            float sqrt_g2 = kAdamEps * em1;
            float g1 = u * (sqrt_g2 + kAdamEps), g2 = sqrt_g2 * sqrt_g2;
            g1 = kBeta1 * g1 + (1.f - kBeta1) * v;
            g2 = kBeta2 * g2 + (1.f - kBeta2) * v * v;
            // the reference builds this kernel with --use_fast_math: approximate division and
            // square root are its own arithmetic here (cmake/SsBackendCuda.cmake:95-102)
            float lr1 = lr_ibc1, c2 = ibc2;
            if (STEPS) {
                // a thread's four cells belong to one splat, or to two neighbours: the two powers are taken once per splat
                const int64_t splat = idx / stride;
                if (splat != step_splat) {
                    step_splat = splat;
                    const float step = (float)steps[splat];
                    step_lr1 = lr * inv_bias_correction(kBeta1, step);
                    step_c2 = inv_bias_correction(kBeta2, step);
                }
                lr1 = step_lr1; c2 = step_c2;
            }
            xv -= __fdividef(lr1 * g1, sqrt_approx(g2 * c2) + kAdamEps);
            float sq = sqrt_approx(fmaxf(g2, 0.0f));
            u_new[k] = __fdividef(g1, sq + kAdamEps);
            float y = sq * (1.0f / kAdamEps);
            s_new[k] = __logf(y > 1.0e6f ? y : 1.0f + y);      // log(1) = 0 exactly for a cell that never saw a gradient
            x[k] = xv;
        }
    }
    float mn[3] = {1e30f, 1e30f, 1e30f}, mx[3] = {-1e30f, -1e30f, -1e30f};
#pragma unroll
    for (int k = 0; k < 4; ++k)
        if (inside[k]) {
            mn[0] = fminf(mn[0], x[k]); mx[0] = fmaxf(mx[0], x[k]);
            mn[1] = fminf(mn[1], u_new[k]); mx[1] = fmaxf(mx[1], u_new[k]);
            mn[2] = fminf(mn[2], s_new[k]); mx[2] = fmaxf(mx[2], s_new[k]);
        }
    {
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
        uint32_t r[6];
#pragma unroll
        for (int k = 0; k < 3; ++k) { r[k] = __reduce_min_sync(0xffffffffu, f2ord(mn[k])); r[3 + k] = __reduce_max_sync(0xffffffffu, f2ord(mx[k])); }
        if (lane == 0) {
#pragma unroll
            for (int k = 0; k < 6; ++k) sh[k][w] = r[k];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            mn[k] = ord2f(min(sh[k][0], sh[k][1]));
            mx[k] = ord2f(max(sh[3 + k][0], sh[3 + k][1]));
        }
    }
    const float vmin = mn[0], vmax = mx[0], umin = mn[1], umax = mx[1], smin = mn[2], smax = mx[2];
    const float vscale = __fdividef(vq, fmaxf(vmax - vmin, 1e-30f));
    const float uscale = __fdividef(oq, fmaxf(umax - umin, kAdamEps)), sscale = __fdividef(oq, fmaxf(smax - smin, kAdamEps));
    uint32_t vout[4], oout[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        vout[k] = kPlainValue ? __float_as_uint(x[k]) : (uint32_t)fminf(fmaxf(rintf((x[k] - vmin) * vscale), 0.0f), vq);
        uint32_t uqc = (uint32_t)fminf(fmaxf(rintf((u_new[k] - umin) * uscale), 0.0f), oq);
        uint32_t sqc = (uint32_t)fminf(fmaxf(rintf((s_new[k] - smin) * sscale), 0.0f), oq);
        oout[k] = kNibbles ? (uqc | (sqc << 4)) : (uqc | (sqc << 8));
    }
    const int64_t (&vdisp)[SSB_MAX_PEERS - 1] = kPlainValue ? po.params : po.sh_packed;
    const int64_t vmc = kPlainValue ? po.mc_params : po.mc_sh_packed;
    if (full) {
        if (kPlainValue) store_all<PEER>((uint4*)((float*)value_packed + idx0), make_uint4(vout[0], vout[1], vout[2], vout[3]), po, vdisp, vmc);
        else if (VALUE_BITS == 16) store_all<PEER>((ushort4*)((uint16_t*)value_packed + idx0), make_ushort4(vout[0], vout[1], vout[2], vout[3]), po, vdisp, vmc);
        else store_all<PEER>((uchar4*)(value_packed + idx0), make_uchar4(vout[0], vout[1], vout[2], vout[3]), po, vdisp, vmc);
        if (kNibbles) *(uint32_t*)(optim_packed + idx0) = oout[0] | (oout[1] << 8) | (oout[2] << 16) | (oout[3] << 24);
        else *(uint2*)(optim_packed + 2 * idx0) = make_uint2(oout[0] | (oout[1] << 16), oout[2] | (oout[3] << 16));
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (inside[k]) {
                const int64_t idx = idx0 + k;
                if (kPlainValue) store_all<PEER>((uint32_t*)value_packed + idx, vout[k], po, vdisp, vmc);
                else if (VALUE_BITS == 8) store_all<PEER>(value_packed + idx, (uint8_t)vout[k], po, vdisp);
                else store_all<PEER>((uint16_t*)value_packed + idx, (uint16_t)vout[k], po, vdisp);
                if (kNibbles) optim_packed[idx] = (uint8_t)oout[k];
                else { optim_packed[2 * idx] = (uint8_t)(oout[k] & 255u); optim_packed[2 * idx + 1] = (uint8_t)(oout[k] >> 8); }
            }
    }
    if (threadIdx.x == 0) {
        if (!kPlainValue) store_all<PEER>(value_bounds + blk, make_float2(vmin, vmax), po, po.sh_bounds, po.mc_sh_bounds);
        optim_bounds[blk] = make_float4(umin, umax, smin, smax);
    }
}

// The same update on the layouts of the reference's fused backward + optimiser at quantisation level 1
// (src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:709-975): one float4 of state bounds and one float2 of value bounds
// per 256 SPLATS, covering all 45 cells of each; 8-bit joint state codes; 8- or 16-bit values.  One CTA per block of 256
// splats = 11520 cells, 18 per thread, a thread's cells 640 apart so that every load and store of a warp is contiguous; the
// updated value and the two new state coordinates of a thread's cells wait in registers for the block's new bounds.
// n_active: live cells per splat (3 * coefficients of the active SH degree); the others are not updated but written as zero
// value and zero moments against bounds widened to contain zero (the SH degree warm-up, :836-857, :918-925).
constexpr int kSbThreads = 640, kSbCells = 256 * 45, kSbPer = kSbCells / kSbThreads;
static_assert(kSbPer * kSbThreads == kSbCells, "a block's cells divide evenly over the CTA");

template <int VALUE_BITS, bool STEPS>
__global__ void __launch_bounds__(kSbThreads, 1) adam_sh_splat_block_kernel(
    float* __restrict__ grad, uint8_t* __restrict__ optim_packed, float4* __restrict__ optim_bounds, uint8_t* __restrict__ value_packed,
    float2* __restrict__ value_bounds, int64_t first_block, int64_t n_total_splats, int n_active, float lr_ibc1, float ibc2, float decay,
    float grad_scale, int zero_grad, const int32_t* __restrict__ steps, float lr) {
    __shared__ uint32_t red[6][kSbThreads / 32];
    __shared__ float2 step_terms[STEPS ? 256 : 1];      // per splat of the block: lr / (1 - beta1^t), 1 / (1 - beta2^t)
    const int64_t blk = first_block + blockIdx.x;
    const int64_t cell0 = blk * kSbCells;
    const int n_cells = (int)min((int64_t)kSbCells, (n_total_splats - blk * 256) * 45);
    if (STEPS) {
        if (threadIdx.x < 256 && threadIdx.x * 45 < n_cells) {
            const float step = (float)steps[blk * 256 + threadIdx.x];
            step_terms[threadIdx.x] = make_float2(lr * inv_bias_correction(kBeta1, step), inv_bias_correction(kBeta2, step));
        }
        __syncthreads();
    }
    constexpr float vq = (float)((1u << VALUE_BITS) - 1u), vinv = 1.0f / vq;
    const float oq = 255.0f, oinv = 1.0f / 255.0f;
    const float2 vmm = value_bounds[blk];
    const float4 omm = optim_bounds[blk];
    float x[kSbPer], u_new[kSbPer], s_new[kSbPer];
    float mn[3] = {1e30f, 1e30f, 1e30f}, mx[3] = {-1e30f, -1e30f, -1e30f};
#pragma unroll
    for (int k = 0; k < kSbPer; ++k) {
        const int c = threadIdx.x + k * kSbThreads;
        x[k] = u_new[k] = s_new[k] = 0.f;
        const int splat = c / 45;
        if (c < n_cells && c - splat * 45 < n_active) {
            const int64_t idx = cell0 + c;
            float v = grad[idx];
            if (zero_grad) grad[idx] = 0.f;
            const uint32_t vcode = VALUE_BITS == 8 ? (uint32_t)value_packed[idx] : (uint32_t)((const uint16_t*)value_packed)[idx];
            const uint32_t oc = ((const uint16_t*)optim_packed)[idx];
            float xv = vmm.x + (vmm.y - vmm.x) * ((float)vcode * vinv);
            if (!isfinite(v)) v = 0.f;
            v *= grad_scale;
            v += decay * xv;
            const float u = omm.x + (omm.y - omm.x) * ((float)(oc & 255u) * oinv);
            const float ls = omm.z + (omm.w - omm.z) * ((float)(oc >> 8) * oinv);
            const float em1 = __expf(ls) - 1.0f;          // exact at 0; see adam_qq_kernel
            const float sqrt_g2 = kAdamEps * em1;
            float g1 = u * (sqrt_g2 + kAdamEps), g2 = sqrt_g2 * sqrt_g2;
            g1 = kBeta1 * g1 + (1.f - kBeta1) * v;
            g2 = kBeta2 * g2 + (1.f - kBeta2) * v * v;
            float lr1 = lr_ibc1, c2 = ibc2;
            if (STEPS) { const float2 t = step_terms[splat]; lr1 = t.x; c2 = t.y; }
            xv -= __fdividef(lr1 * g1, sqrt_approx(g2 * c2) + kAdamEps);
            const float sq = sqrt_approx(fmaxf(g2, 0.0f));
            u_new[k] = __fdividef(g1, sq + kAdamEps);
            const float y = sq * (1.0f / kAdamEps);
            s_new[k] = __logf(y > 1.0e6f ? y : 1.0f + y);      // log(1) = 0 exactly for a cell that never saw a gradient
            x[k] = xv;
            mn[0] = fminf(mn[0], xv); mx[0] = fmaxf(mx[0], xv);
            mn[1] = fminf(mn[1], u_new[k]); mx[1] = fmaxf(mx[1], u_new[k]);
            mn[2] = fminf(mn[2], s_new[k]); mx[2] = fmaxf(mx[2], s_new[k]);
        }
    }
    {
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
        uint32_t r[6];
#pragma unroll
        for (int k = 0; k < 3; ++k) { r[k] = __reduce_min_sync(0xffffffffu, f2ord(mn[k])); r[3 + k] = __reduce_max_sync(0xffffffffu, f2ord(mx[k])); }
        if (lane == 0) {
#pragma unroll
            for (int k = 0; k < 6; ++k) red[k][w] = r[k];
        }
        __syncthreads();
        if (w == 0) {
#pragma unroll
            for (int k = 0; k < 6; ++k) {
                const uint32_t mine = lane < kSbThreads / 32 ? red[k][lane] : (k < 3 ? 0xffffffffu : 0u);
                r[k] = k < 3 ? __reduce_min_sync(0xffffffffu, mine) : __reduce_max_sync(0xffffffffu, mine);
            }
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int k = 0; k < 6; ++k) red[k][0] = r[k];
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 3; ++k) { mn[k] = ord2f(red[k][0]); mx[k] = ord2f(red[3 + k][0]); }
    }
    if (n_active < 45) {       // zero must be representable: the idle cells are written as zero
        mn[0] = fminf(mn[0], 0.f); mx[0] = fmaxf(mx[0], 0.f);
        mn[1] = fminf(mn[1], 0.f); mx[1] = fmaxf(mx[1], 0.f);
        mn[2] = fminf(mn[2], 0.f);
    }
    const float vmin = mn[0], vmax = mx[0], umin = mn[1], umax = mx[1], smin = mn[2], smax = mx[2];
    const float vscale = __fdividef(vq, fmaxf(vmax - vmin, 1e-30f));
    const float uscale = __fdividef(oq, fmaxf(umax - umin, kAdamEps)), sscale = __fdividef(oq, fmaxf(smax - smin, kAdamEps));
#pragma unroll
    for (int k = 0; k < kSbPer; ++k) {
        const int c = threadIdx.x + k * kSbThreads;
        if (c < n_cells) {
            const int64_t idx = cell0 + c;
            // an idle cell holds x = u = s = 0 here
            const uint32_t vout = (uint32_t)fminf(fmaxf(rintf((x[k] - vmin) * vscale), 0.0f), vq);
            const uint32_t uqc = (uint32_t)fminf(fmaxf(rintf((u_new[k] - umin) * uscale), 0.0f), oq);
            const uint32_t sqc = (uint32_t)fminf(fmaxf(rintf((s_new[k] - smin) * sscale), 0.0f), oq);
            if (VALUE_BITS == 8) value_packed[idx] = (uint8_t)vout; else ((uint16_t*)value_packed)[idx] = (uint16_t)vout;
            ((uint16_t*)optim_packed)[idx] = (uint16_t)(uqc | (sqc << 8));
        }
    }
    if (threadIdx.x == 0) {
        value_bounds[blk] = make_float2(vmin, vmax);
        optim_bounds[blk] = make_float4(umin, umax, smin, smax);
    }
}

template <int BITS>
__global__ void __launch_bounds__(256) quant_encode_kernel(const float* __restrict__ values, int64_t numel, uint8_t* __restrict__ packed, float2* __restrict__ bounds) {
    __shared__ uint32_t sh[2][8];
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const bool inside = idx < numel;
    float v = inside ? values[idx] : 0.f;
    const float mn_in[1] = {inside ? v : 1e30f}, mx_in[1] = {inside ? v : -1e30f};
    float mn_o[1], mx_o[1];
    block_minmax<1, 1>(mn_in, mx_in, mn_o, mx_o, sh);
    const float mn = mn_o[0], mx = mx_o[0];
    constexpr float qmax = (float)((1 << BITS) - 1);
    if (inside) {
        float range = fmaxf(mx - mn, 1e-30f);
        float qf = fminf(fmaxf(roundf(qmax * (v - mn) / range), 0.0f), qmax);
        if (BITS == 8) packed[idx] = (uint8_t)qf; else ((uint16_t*)packed)[idx] = (uint16_t)qf;
    }
    if (threadIdx.x == 0) bounds[blockIdx.x] = make_float2(mn, mx);
}

template <int BITS>
__global__ void __launch_bounds__(256) quant_decode_kernel(const uint8_t* __restrict__ packed, const float2* __restrict__ bounds, int64_t numel, float* __restrict__ values) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= numel) return;
    float2 mm = bounds[idx >> 8];
    float q = BITS == 8 ? (float)packed[idx] : (float)((const uint16_t*)packed)[idx];
    values[idx] = mm.x + (mm.y - mm.x) * (q * (1.0f / (float)((1 << BITS) - 1)));
}

}  // namespace ssb

namespace ssb {

static int moments_q16_of(const SsbMomentsQ16* moments, MomentsQ16* out) {
    for (int t = 0; t < 5; ++t) {
        SSB_REQUIRE(moments->d_packed[t] && moments->d_bounds[t], "16-bit moments: array %d missing", t);
        out->packed[t] = moments->d_packed[t];
        out->bounds[t] = (float4*)moments->d_bounds[t];
    }
    return SSB_OK;
}

static int adam_step_impl(const SsbSplats* params, const SsbSplats* grads, const SsbSplats* m1, const SsbSplats* m2,
                          int64_t first, int64_t count, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, const PeerOffsets* peers,
                          void* stream, const MomentsQ16* nq = nullptr) {
    // nq: the moments of the five non-SH arrays are 16-bit codes (m1 / m2 then only carry features_sh, if that is fp32)
    SSB_REQUIRE(params && grads && cfg && (nq || (m1 && m2)), "ssb_adam_step: NULL argument");
    SSB_REQUIRE(!nq || count == 0 || first % 256 == 0, "ssb_adam_step: with 16-bit moments the range must start on a multiple of 256 splats");
    SSB_REQUIRE(first >= 0 && count >= 0, "ssb_adam_step: bad range");
    SSB_REQUIRE(cfg->step >= 1, "ssb_adam_step: step must be >= 1 (got %d)", cfg->step);
    if (extras) {
        SSB_REQUIRE(extras->n_total >= first + count, "ssb_adam_step_ex: n_total %lld is smaller than the range's end", (long long)extras->n_total);
        SSB_REQUIRE(!extras->use_scale_agnostic_mean || extras->d_radii, "ssb_adam_step_ex: the scale-agnostic mean update needs d_radii");
    }
    if (count == 0) return SSB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const float ibc1 = 1.0f / (1.0f - powf(kBeta1, (float)cfg->step));
    const float ibc2 = 1.0f / (1.0f - powf(kBeta2, (float)cfg->step));
    // decay = 2 * l2_reg / numel of the whole tensor (fused_adam_step, FusedAppearanceOptim.cu:85); without
    // extras->n_total the whole tensor is taken to be this call's range
    const int64_t n_whole = extras ? extras->n_total : count;
    // with 16-bit moments the reference applies sh_reg_weight to DC undivided (FusedGeometryOptim.cu:343-345)
    const float dc_decay = nq ? cfg->sh_reg_weight : 2.0f * cfg->sh_reg_weight / (float)(n_whole * 3);
    const unsigned blocks = (unsigned)ceil_div(count, 256);
    const PeerOffsets none = {};
    const SsbAdamExtras no_extras = {};
    const SsbSplats no_moments{};
    // multicast mode is built for the plain launch only; the optional parts use per-peer loads and stores
    const bool mc = peers && peers->mc_grads != 0 && peers->mc_params != 0;
    if (nq) {
#define SSB_GEOQ(EX, PEER) adam_geometry_kernel<EX, PEER, true><<<blocks, 256, 0, st>>>(*params, *grads, no_moments, no_moments, first, count, *cfg, ibc1, ibc2, \
                                                                                   dc_decay, EX ? *extras : no_extras, PEER ? *peers : none, *nq)
        if (extras) { if (peers) SSB_GEOQ(true, 1); else SSB_GEOQ(true, 0); }
        else { if (peers) SSB_GEOQ(false, 1); else SSB_GEOQ(false, 0); }
#undef SSB_GEOQ
    } else {
#define SSB_GEO(EX, PEER) adam_geometry_kernel<EX, PEER><<<blocks, 256, 0, st>>>(*params, *grads, *m1, *m2, first, count, *cfg, ibc1, ibc2, dc_decay, \
                                                                            EX ? *extras : no_extras, PEER ? *peers : none)
        if (extras) { if (peers) SSB_GEO(true, 1); else SSB_GEO(true, 0); }
        else { if (mc) SSB_GEO(false, 2); else if (peers) SSB_GEO(false, 1); else SSB_GEO(false, 0); }
#undef SSB_GEO
    }
    SSB_LAUNCHED("adam_geometry_kernel");
    if (params->features_sh) {
        SSB_REQUIRE(grads->features_sh && m1 && m2 && m1->features_sh && m2->features_sh, "ssb_adam_step: SH gradient/moment arrays missing");
        int64_t numel = count * 3 * kNumSh, off = first * 3 * kNumSh;
        const float sh_decay = 2.0f * cfg->sh_reg_weight / (float)(n_whole * 3 * kNumSh);
        const int32_t* steps = extras && extras->d_steps ? extras->d_steps + first : nullptr;
        const unsigned pblocks = (unsigned)ceil_div(ceil_div(numel, 4), 256);
#define SSB_PLAIN(PEER) adam_plain_kernel<PEER><<<pblocks, 256, 0, st>>>( \
            params->features_sh + off, grads->features_sh + off, m1->features_sh + off, m2->features_sh + off, numel, \
            cfg->lr_features_sh * ibc1, ibc2, sh_decay, 0.0f, cfg->grad_scale, cfg->zero_grad, steps, 3 * kNumSh, cfg->lr_features_sh, PEER ? *peers : none)
        if (mc && !steps) SSB_PLAIN(2); else if (peers) SSB_PLAIN(1); else SSB_PLAIN(0);
#undef SSB_PLAIN
        SSB_LAUNCHED("adam_plain_kernel");
    }
    return SSB_OK;
}

static int adam_sh_quantized_impl(float* d_grad, uint8_t* d_optim_packed, float* d_optim_bounds,
                                  void* d_value_packed, float* d_value_bounds, int32_t value_bits, int32_t optim_bits,
                                  int64_t first_cell, int64_t numel, int64_t numel_total,
                                  const SsbAdamConfig* cfg, const int32_t* d_steps, int32_t cells_per_splat, const PeerOffsets* peers, void* stream) {
    SSB_REQUIRE(d_grad && d_optim_packed && d_optim_bounds && d_value_packed && cfg, "ssb_adam_step_sh_quantized: NULL argument");
    SSB_REQUIRE(value_bits == 8 || value_bits == 16 || value_bits == 32, "ssb_adam_step_sh_quantized: value_bits must be 8, 16 or 32 (got %d)", value_bits);
    SSB_REQUIRE(value_bits == 32 || d_value_bounds, "ssb_adam_step_sh_quantized: packed values need a bounds table");
    SSB_REQUIRE(first_cell >= 0 && (first_cell % 256) == 0 && numel >= 0 && first_cell + numel <= numel_total, "ssb_adam_step_sh_quantized: bad cell range");
    SSB_REQUIRE(cfg->step >= 1, "ssb_adam_step_sh_quantized: step must be >= 1");
    SSB_REQUIRE(optim_bits == 4 || optim_bits == 8, "ssb_adam_step_sh_quantized_ex: optim_bits must be 4 or 8 (got %d)", optim_bits);
    SSB_REQUIRE(!d_steps || cells_per_splat >= 1, "ssb_adam_step_sh_quantized_ex: cells_per_splat must be >= 1");
    if (numel == 0) return SSB_OK;
    const float ibc1 = 1.0f / (1.0f - powf(kBeta1, (float)cfg->step));
    const float ibc2 = 1.0f / (1.0f - powf(kBeta2, (float)cfg->step));
    const float decay = 2.0f * cfg->sh_reg_weight / (float)numel_total;
    unsigned blocks = (unsigned)ceil_div(numel, 256);
    int64_t end_total = first_cell + numel;   // cells beyond the range belong to another caller
    const PeerOffsets none = {};
#define SSB_QQ_ARGS(PEER) d_grad, d_optim_packed, (float4*)d_optim_bounds, (uint8_t*)d_value_packed, (float2*)d_value_bounds, first_cell / 256, end_total, \
        cfg->lr_features_sh * ibc1, ibc2, decay, 0.0f, cfg->grad_scale, cfg->zero_grad, d_steps, cells_per_splat, cfg->lr_features_sh, PEER ? *peers : none
#define SSB_QQ_LAUNCH(OB, ST, PEER) \
    do { \
        if (value_bits == 32) adam_qq_kernel<32, OB, ST, PEER><<<blocks, 64, 0, (cudaStream_t)stream>>>(SSB_QQ_ARGS(PEER)); \
        else if (value_bits == 8) adam_qq_kernel<8, OB, ST, PEER><<<blocks, 64, 0, (cudaStream_t)stream>>>(SSB_QQ_ARGS(PEER)); \
        else adam_qq_kernel<16, OB, ST, PEER><<<blocks, 64, 0, (cudaStream_t)stream>>>(SSB_QQ_ARGS(PEER)); \
    } while (0)
#define SSB_QQ_PEER(OB, ST) do { if (peers) SSB_QQ_LAUNCH(OB, ST, 1); else SSB_QQ_LAUNCH(OB, ST, 0); } while (0)
    // multicast mode is built for the default state layout (8-bit state, one step counter) only
    const bool mc = peers && peers->mc_grads != 0 && (value_bits == 32 ? peers->mc_params != 0 : (peers->mc_sh_packed != 0 && peers->mc_sh_bounds != 0));
    if (d_steps) { if (optim_bits == 4) SSB_QQ_PEER(4, true); else SSB_QQ_PEER(8, true); }
    else if (optim_bits == 4) SSB_QQ_PEER(4, false);
    else if (mc) SSB_QQ_LAUNCH(8, false, 2);
    else SSB_QQ_PEER(8, false);
#undef SSB_QQ_PEER
#undef SSB_QQ_LAUNCH
#undef SSB_QQ_ARGS
    SSB_LAUNCHED("adam_qq_kernel");
    return SSB_OK;
}

// Displacements from this rank's copy of each exchanged buffer to the other ranks' copies.
static int peer_offsets(const SsbPeerReplicas* r, bool quantised, PeerOffsets* out) {
    SSB_REQUIRE(r->world >= 1 && r->world <= SSB_MAX_PEERS && r->self >= 0 && r->self < r->world,
                "ssb_reduce_adam_broadcast: bad world/self (%d, %d)", r->world, r->self);
    PeerOffsets po = {};
    for (int p = 0; p < r->world; ++p) {
        SSB_REQUIRE(r->grads[p] && r->params[p], "ssb_reduce_adam_broadcast: rank %d's gradient or parameter buffer is NULL", p);
        SSB_REQUIRE((((uintptr_t)r->grads[p] | (uintptr_t)r->params[p]) & 15) == 0, "ssb_reduce_adam_broadcast: rank %d's buffers must be 16-byte aligned", p);
        SSB_REQUIRE(!quantised || (r->sh_packed[p] && r->sh_bounds[p] && (((uintptr_t)r->sh_packed[p] | (uintptr_t)r->sh_bounds[p]) & 15) == 0),
                    "ssb_reduce_adam_broadcast: rank %d's packed SH buffers are NULL or not 16-byte aligned", p);
        if (p == r->self) continue;
        const int k = po.n++;
        po.grads[k] = (int64_t)((char*)r->grads[p] - (char*)r->grads[r->self]);
        po.params[k] = (int64_t)((char*)r->params[p] - (char*)r->params[r->self]);
        if (quantised) {
            po.sh_packed[k] = (int64_t)((char*)r->sh_packed[p] - (char*)r->sh_packed[r->self]);
            po.sh_bounds[k] = (int64_t)((char*)r->sh_bounds[p] - (char*)r->sh_bounds[r->self]);
        }
    }
    // multicast addresses: used only when every exchanged buffer has one
    const bool mc = r->mc_grads && r->mc_params && (!quantised || (r->mc_sh_packed && r->mc_sh_bounds)) && r->world > 1;
    if (mc) {
        SSB_REQUIRE((((uintptr_t)r->mc_grads | (uintptr_t)r->mc_params | (uintptr_t)r->mc_sh_packed | (uintptr_t)r->mc_sh_bounds) & 15) == 0,
                    "ssb_reduce_adam_broadcast: multicast addresses must be 16-byte aligned");
        po.mc_grads = (int64_t)((char*)r->mc_grads - (char*)r->grads[r->self]);
        po.mc_params = (int64_t)((char*)r->mc_params - (char*)r->params[r->self]);
        if (quantised) {
            po.mc_sh_packed = (int64_t)((char*)r->mc_sh_packed - (char*)r->sh_packed[r->self]);
            po.mc_sh_bounds = (int64_t)((char*)r->mc_sh_bounds - (char*)r->sh_bounds[r->self]);
        }
    }
    *out = po;
    return SSB_OK;
}

}  // namespace ssb

extern "C" {

int ssb_adam_step(const SsbSplats* params, const SsbSplats* grads, const SsbSplats* m1, const SsbSplats* m2,
                  int64_t first, int64_t count, const SsbAdamConfig* cfg, void* stream) {
    return ssb::adam_step_impl(params, grads, m1, m2, first, count, cfg, nullptr, nullptr, stream);
}

int ssb_adam_step_ex(const SsbSplats* params, const SsbSplats* grads, const SsbSplats* m1, const SsbSplats* m2,
                     int64_t first, int64_t count, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream) {
    return ssb::adam_step_impl(params, grads, m1, m2, first, count, cfg, extras, nullptr, stream);
}

int ssb_adam_step_q16(const SsbSplats* params, const SsbSplats* grads, const SsbMomentsQ16* moments, int64_t first, int64_t count,
                      const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(params && grads && moments && cfg, "ssb_adam_step_q16: NULL argument");
    SSB_REQUIRE(params->means && params->quats && params->scales && params->opacities && params->features_dc, "ssb_adam_step_q16: parameter arrays missing");
    SSB_REQUIRE(grads->means && grads->quats && grads->scales && grads->opacities && grads->features_dc, "ssb_adam_step_q16: gradient arrays missing");
    MomentsQ16 nq;
    if (int e = moments_q16_of(moments, &nq)) return e;
    // features_sh is not this call's business: the caller steps it with ssb_adam_plain or ssb_adam_step_sh_quantized
    SsbSplats p = *params, g = *grads;
    p.features_sh = nullptr; g.features_sh = nullptr;
    return adam_step_impl(&p, &g, nullptr, nullptr, first, count, cfg, extras, nullptr, stream, &nq);
}

int ssb_adam_step_sh_splat_blocks(float* d_grad, uint8_t* d_optim_packed, float* d_optim_bounds, void* d_value_packed, float* d_value_bounds,
                                  int32_t value_bits, int64_t first_splat, int64_t n_splats, int64_t n_total, int32_t active_sh_degree_plus1,
                                  const SsbAdamConfig* cfg, const int32_t* d_steps, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_grad && d_optim_packed && d_optim_bounds && d_value_packed && d_value_bounds && cfg, "ssb_adam_step_sh_splat_blocks: NULL argument");
    SSB_REQUIRE(value_bits == 8 || value_bits == 16, "ssb_adam_step_sh_splat_blocks: value_bits must be 8 or 16 (got %d)", value_bits);
    SSB_REQUIRE(first_splat >= 0 && (first_splat % 256) == 0 && n_splats >= 0 && first_splat + n_splats <= n_total,
                "ssb_adam_step_sh_splat_blocks: bad splat range (the first splat must be a multiple of 256)");
    SSB_REQUIRE(active_sh_degree_plus1 >= 0 && active_sh_degree_plus1 <= 4, "ssb_adam_step_sh_splat_blocks: SH degree + 1 must be 0..4 (got %d)", active_sh_degree_plus1);
    SSB_REQUIRE(cfg->step >= 1 || d_steps, "ssb_adam_step_sh_splat_blocks: step must be >= 1");
    SSB_REQUIRE(((uintptr_t)d_optim_packed & 1) == 0 && ((uintptr_t)d_value_packed & 1) == 0, "ssb_adam_step_sh_splat_blocks: code buffers must be 2-byte aligned");
    const int degree = active_sh_degree_plus1 == 0 ? 3 : active_sh_degree_plus1 - 1;
    const int n_active = 3 * (degree * (degree + 2));
    if (n_splats == 0 || n_active == 0) return SSB_OK;     // at degree 0 the reference's kernel has no SH section
    const int step = cfg->step >= 1 ? cfg->step : 1;
    const float ibc1 = 1.0f / (1.0f - powf(kBeta1, (float)step)), ibc2 = 1.0f / (1.0f - powf(kBeta2, (float)step));
    const float decay = 2.0f * cfg->sh_reg_weight / (float)(n_total * 45);
    const unsigned blocks = (unsigned)ceil_div(n_splats, 256);
    // a range that ends inside a block would leave that block's other splats with bounds that no longer fit their codes
    SSB_REQUIRE((n_splats % 256) == 0 || first_splat + n_splats == n_total, "ssb_adam_step_sh_splat_blocks: a range ends on a multiple of 256 splats or at the last splat");
#define SSB_SB_ARGS d_grad, d_optim_packed, (float4*)d_optim_bounds, (uint8_t*)d_value_packed, (float2*)d_value_bounds, first_splat / 256, n_total, n_active, \
        cfg->lr_features_sh * ibc1, ibc2, decay, cfg->grad_scale, cfg->zero_grad, d_steps, cfg->lr_features_sh
    cudaStream_t st = (cudaStream_t)stream;
    if (value_bits == 16) { if (d_steps) adam_sh_splat_block_kernel<16, true><<<blocks, kSbThreads, 0, st>>>(SSB_SB_ARGS); else adam_sh_splat_block_kernel<16, false><<<blocks, kSbThreads, 0, st>>>(SSB_SB_ARGS); }
    else { if (d_steps) adam_sh_splat_block_kernel<8, true><<<blocks, kSbThreads, 0, st>>>(SSB_SB_ARGS); else adam_sh_splat_block_kernel<8, false><<<blocks, kSbThreads, 0, st>>>(SSB_SB_ARGS); }
#undef SSB_SB_ARGS
    SSB_LAUNCHED("adam_sh_splat_block_kernel");
    return SSB_OK;
}

int ssb_adam_plain(float* d_param, float* d_grad, float* d_m1, float* d_m2, int64_t numel, int32_t stride, float lr, int32_t step,
                   const int32_t* d_steps, float l2_reg, float l2_reg_offset, float grad_scale, int32_t zero_grad, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_param && d_grad && d_m1 && d_m2, "ssb_adam_plain: NULL argument");
    SSB_REQUIRE(numel >= 0 && stride > 0 && (d_steps || step >= 1), "ssb_adam_plain: bad sizes or step");
    if (numel == 0) return SSB_OK;
    const float ibc1 = d_steps ? 1.f : 1.0f / (1.0f - powf(kBeta1, (float)step)), ibc2 = d_steps ? 1.f : 1.0f / (1.0f - powf(kBeta2, (float)step));
    const float decay = 2.0f * l2_reg / (float)numel;            // fused_adam_step, src/kernels/optim/FusedAppearanceOptim.cu:85
    adam_plain_kernel<0><<<(unsigned)ceil_div(ceil_div(numel, 4), 256), 256, 0, (cudaStream_t)stream>>>(
        d_param, d_grad, d_m1, d_m2, numel, lr * ibc1, ibc2, decay, l2_reg_offset, grad_scale, zero_grad, d_steps, stride, lr, PeerOffsets{});
    SSB_LAUNCHED("adam_plain_kernel");
    return SSB_OK;
}

int ssb_adam_step_sh_quantized(float* d_grad, uint8_t* d_optim_packed, float* d_optim_bounds,
                               void* d_value_packed, float* d_value_bounds, int32_t value_bits,
                               int64_t first_cell, int64_t numel, int64_t numel_total,
                               const SsbAdamConfig* cfg, void* stream) {
    return ssb::adam_sh_quantized_impl(d_grad, d_optim_packed, d_optim_bounds, d_value_packed, d_value_bounds, value_bits, 8, first_cell, numel,
                                       numel_total, cfg, nullptr, 1, nullptr, stream);
}

int ssb_adam_step_sh_quantized_ex(float* d_grad, uint8_t* d_optim_packed, float* d_optim_bounds,
                                  void* d_value_packed, float* d_value_bounds, int32_t value_bits, int32_t optim_bits,
                                  int64_t first_cell, int64_t numel, int64_t numel_total,
                                  const SsbAdamConfig* cfg, const int32_t* d_steps, int32_t cells_per_splat, void* stream) {
    return ssb::adam_sh_quantized_impl(d_grad, d_optim_packed, d_optim_bounds, d_value_packed, d_value_bounds, value_bits, optim_bits, first_cell,
                                       numel, numel_total, cfg, d_steps, cells_per_splat, nullptr, stream);
}

static int reduce_adam_broadcast_impl(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                                      const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                                      int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream,
                                      const SsbMomentsQ16* moments_q16) {
    using namespace ssb;
    SSB_REQUIRE(replicas && params && grads && cfg && (moments_q16 || (m1 && m2)), "ssb_reduce_adam_broadcast: NULL argument");
    MomentsQ16 nq;
    if (moments_q16) {
        if (int e = moments_q16_of(moments_q16, &nq)) return e;
        SSB_REQUIRE(count == 0 || first % 256 == 0, "ssb_reduce_adam_broadcast_q16: a rank's range must start on a multiple of 256 splats");
    }
    SSB_REQUIRE(first >= 0 && count >= 0 && first + count <= n_total, "ssb_reduce_adam_broadcast: bad splat range");
    const bool quantised = sh_state != nullptr;
    SSB_REQUIRE(quantised == (params->features_sh == nullptr), "ssb_reduce_adam_broadcast: give either fp32 SH inside params or an SsbShAdamState");
    PeerOffsets po;
    if (int e = peer_offsets(replicas, quantised && sh_state->value_bits != 32, &po)) return e;
    // everything the kernels address through a displacement must lie behind this rank's base of that buffer
    const char* gbase = (const char*)replicas->grads[replicas->self];
    const char* pbase = (const char*)replicas->params[replicas->self];
    const float* g_arrays[6] = {grads->means, grads->quats, grads->scales, grads->opacities, grads->features_dc, grads->features_sh};
    const float* p_arrays[6] = {params->means, params->quats, params->scales, params->opacities, params->features_dc, params->features_sh};
    for (int k = 0; k < 6; ++k) {
        SSB_REQUIRE(g_arrays[k] != nullptr && (const char*)g_arrays[k] >= gbase, "ssb_reduce_adam_broadcast: gradient array %d is not inside the exchanged gradient buffer", k);
        SSB_REQUIRE(k == 5 ? (quantised || (const char*)p_arrays[k] >= pbase) : (p_arrays[k] != nullptr && (const char*)p_arrays[k] >= pbase),
                    "ssb_reduce_adam_broadcast: parameter array %d is not inside the exchanged parameter buffer", k);
    }
    if (quantised) {
        SSB_REQUIRE(sh_state->d_optim_packed && sh_state->d_optim_bounds && sh_state->d_value_packed, "ssb_reduce_adam_broadcast: NULL SH state");
        SSB_REQUIRE(sh_state->layout == SSB_SH_LAYOUT_CELL_BLOCKS, "ssb_reduce_adam_broadcast: the SH state must be in the cell-block layout");
        SSB_REQUIRE(sh_state->value_bits == 32 || (sh_state->d_value_packed == replicas->sh_packed[replicas->self] &&
                                                   (void*)sh_state->d_value_bounds == replicas->sh_bounds[replicas->self]),
                    "ssb_reduce_adam_broadcast: the packed SH values and bounds must be this rank's exchanged buffers");
        SSB_REQUIRE((first * 3 * kNumSh) % 256 == 0 && (((first + count) * 3 * kNumSh) % 256 == 0 || first + count == n_total),
                    "ssb_reduce_adam_broadcast: a rank's range must cover whole 256-cell quantisation blocks (splat ranges in multiples of 256)");
    }
    if (moments_q16) { po.mc_grads = 0; po.mc_params = 0; }      // per-peer loads and stores (the multicast kernels keep fp32 moments)
    const PeerOffsets* peers = po.n > 0 ? &po : nullptr;
    if (peers) {
        // the kernels move a CTA's 256 splats of every array with 16-byte accesses
        SSB_REQUIRE((first & 3) == 0, "ssb_reduce_adam_broadcast: with peers a rank's range must start at a multiple of 4 splats");
        for (int k = 0; k < 6; ++k)
            SSB_REQUIRE((((uintptr_t)g_arrays[k] | (uintptr_t)p_arrays[k]) & 15) == 0, "ssb_reduce_adam_broadcast: array %d must be 16-byte aligned", k);
    }
    SsbAdamExtras ex_local;
    const SsbAdamExtras* ex = extras;
    if (!ex && count != n_total) {        // regulariser weights are divided by the model's splat count, not the range's
        ex_local = SsbAdamExtras{};
        ex_local.n_total = n_total;
        ex = cfg->sh_reg_weight != 0.0f ? &ex_local : nullptr;
    }
    if (int e = adam_step_impl(params, grads, m1, m2, first, count, cfg, ex, peers, stream, moments_q16 ? &nq : nullptr)) return e;
    if (quantised) {
        const int32_t* steps = extras ? extras->d_steps : nullptr;
        return adam_sh_quantized_impl(grads->features_sh, sh_state->d_optim_packed, sh_state->d_optim_bounds, sh_state->d_value_packed,
                                      sh_state->d_value_bounds, sh_state->value_bits, sh_state->optim_bits ? sh_state->optim_bits : 8,
                                      first * 3 * kNumSh, count * 3 * kNumSh, n_total * 3 * kNumSh, cfg, steps, 3 * kNumSh, peers, stream);
    }
    return SSB_OK;
}

int ssb_reduce_adam_broadcast(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                              const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                              int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream) {
    SSB_REQUIRE(m1 && m2, "ssb_reduce_adam_broadcast: NULL argument");
    return reduce_adam_broadcast_impl(replicas, params, grads, m1, m2, sh_state, first, count, n_total, cfg, extras, stream, nullptr);
}

int ssb_reduce_adam_broadcast_q16(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                                  const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                                  int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream) {
    SSB_REQUIRE(moments, "ssb_reduce_adam_broadcast_q16: NULL moments");
    return reduce_adam_broadcast_impl(replicas, params, grads, m1, m2, sh_state, first, count, n_total, cfg, extras, stream, moments);
}

static int exchange_step_impl(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                              const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                              int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras,
                              SsbBarrierFn barrier, void* barrier_ctx, void* stream, const SsbMomentsQ16* moments_q16) {
    using namespace ssb;
    SSB_REQUIRE(replicas && barrier, "ssb_exchange_step: NULL argument");
    // every rank's backward passes are complete before anyone reads a partial gradient
    if (barrier(barrier_ctx, stream) != 0) {
        set_error("ssb_exchange_step: a rank did not arrive at the barrier before the exchange; nothing was launched");
        return SSB_ERR_PEER;
    }
    if (int e = reduce_adam_broadcast_impl(replicas, params, grads, m1, m2, sh_state, first, count, n_total, cfg, extras, stream, moments_q16)) return e;
    // every replica is complete before anyone's next forward pass
    if (barrier(barrier_ctx, stream) != 0) {
        set_error("ssb_exchange_step: a rank did not arrive at the barrier after the exchange; replicas may be incomplete");
        return SSB_ERR_PEER;
    }
    return SSB_OK;
}

int ssb_exchange_step(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                      const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                      int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras,
                      SsbBarrierFn barrier, void* barrier_ctx, void* stream) {
    SSB_REQUIRE(m1 && m2, "ssb_exchange_step: NULL argument");
    return exchange_step_impl(replicas, params, grads, m1, m2, sh_state, first, count, n_total, cfg, extras, barrier, barrier_ctx, stream, nullptr);
}

int ssb_exchange_step_q16(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                          const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                          int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras,
                          SsbBarrierFn barrier, void* barrier_ctx, void* stream) {
    SSB_REQUIRE(moments, "ssb_exchange_step_q16: NULL moments");
    return exchange_step_impl(replicas, params, grads, m1, m2, sh_state, first, count, n_total, cfg, extras, barrier, barrier_ctx, stream, moments);
}

int ssb_quant_encode(const float* d_values, int64_t numel, int32_t bits, void* d_packed, float* d_bounds, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_values && d_packed && d_bounds && numel >= 0, "ssb_quant_encode: bad argument");
    SSB_REQUIRE(bits == 8 || bits == 16, "ssb_quant_encode: bits must be 8 or 16 (got %d)", bits);
    if (numel == 0) return SSB_OK;
    unsigned blocks = (unsigned)ceil_div(numel, 256);
    if (bits == 8) quant_encode_kernel<8><<<blocks, 256, 0, (cudaStream_t)stream>>>(d_values, numel, (uint8_t*)d_packed, (float2*)d_bounds);
    else quant_encode_kernel<16><<<blocks, 256, 0, (cudaStream_t)stream>>>(d_values, numel, (uint8_t*)d_packed, (float2*)d_bounds);
    SSB_LAUNCHED("quant_encode_kernel");
    return SSB_OK;
}

int ssb_quant_decode(const void* d_packed, const float* d_bounds, int64_t numel, int32_t bits, float* d_values, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_values && d_packed && d_bounds && numel >= 0, "ssb_quant_decode: bad argument");
    SSB_REQUIRE(bits == 8 || bits == 16, "ssb_quant_decode: bits must be 8 or 16 (got %d)", bits);
    if (numel == 0) return SSB_OK;
    unsigned blocks = (unsigned)ceil_div(numel, 256);
    if (bits == 8) quant_decode_kernel<8><<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)d_packed, (const float2*)d_bounds, numel, d_values);
    else quant_decode_kernel<16><<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)d_packed, (const float2*)d_bounds, numel, d_values);
    SSB_LAUNCHED("quant_decode_kernel");
    return SSB_OK;
}

}  // extern "C"
