// Fused image loss: w_l1 * mean|render - gt| + w_ssim * (1 - SSIM) with its
// gradient with respect to the render, in one kernel.
//
// Restates the RGB-L1 term of the reference's per-pixel loss and its reverse
// (src/shaders/per_pixel_losses.slang:133-176,365-375: v = w * sign(r-g)/(3*B*P))
// and the fused SSIM forward+backward of src/kernels/loss/FusedSSIM.cu:639-1022
// (11-tap Gaussian, sigma 1.5, zero padding, C1 = 1e-4, C2 = 9e-4, gradient
// scale -w_ssim/(3*B*H*W) added on top of the L1 gradient).
//
// One CTA produces a 32x32 block of gradient pixels for all three channels.
// That needs the SSIM partial derivatives of the 42x42 window centres around
// it, hence the moments of a 52x52 input patch: the patch is loaded once per
// channel into shared memory, both separable convolutions run out of shared
// memory, and only the 32x32 gradient block is written.
#include "ssb_common.cuh"

namespace ssb {

constexpr int kLossTile = 32;
constexpr int kHalo = 5;
constexpr int kIn = kLossTile + 4 * kHalo;    // 52: input patch edge
constexpr int kMid = kLossTile + 2 * kHalo;   // 42: window-centre patch edge
constexpr int kLossThreads = 256;

__constant__ float cGaussW[11] = {
    0.001028380123898387f, 0.0075987582094967365f, 0.036000773310661316f, 0.10936068743467331f,
    0.21300552785396576f, 0.26601171493530273f, 0.21300552785396576f, 0.10936068743467331f,
    0.036000773310661316f, 0.0075987582094967365f, 0.001028380123898387f};

// shared memory layout (floats)
// Row strides of the partial maps and of their row convolution are odd (43, 33): step 4 works on two neighbouring outputs
// per thread, so a warp covers two rows with even column offsets, and an even stride would put both rows on the same banks.
constexpr int kDStride = kMid + 1, kHStride = kLossTile + 1;
// Row stride of the row-convolved moments.  Step 3 walks them with one thread per (group of three rows, column): item o reads
// word (o / 42) * 3 * stride + o % 42 + const, which is o + const modulo 32 -- one bank per lane -- when 3 * stride = 42 (mod 32).
constexpr int kMStride = 46;
constexpr int kSmemA = 3 * kMid * kDStride;           // X and Y patches (2*52*52 = 5408); later the 3 partial maps (3*42*43 = 5418)
constexpr int kSmemB = 5 * kIn * kMStride;            // row-convolved moments; later 3*42*33 row-convolved partials
static_assert(kSmemA >= 2 * kIn * kIn && kSmemB >= 3 * kMid * kHStride, "shared-memory aliases must fit");
constexpr int kLossSmemBytes = (kSmemA + kSmemB) * 4;
// With a mask: a sixth moment (the window's coverage) and the 52x52 mask patch, which stays live to the end.
constexpr int kSmemBMasked = 6 * kIn * kMStride;
constexpr int kLossSmemBytesMasked = (kSmemA + kSmemBMasked + kIn * kIn) * 4;

// Which pixels take part (src/kernels/loss/FusedSSIM.cu:105-126, src/core/Interpolation.cuh:108-120): bytes [Bm][Hm][Wm],
// != 0 = takes part; nearest-sampled when the size is not the image's; a tap outside the image reads "takes part".
struct LossMask {
    const uint8_t* mask;
    int Bm, Hm, Wm;
    const unsigned long long* total;   // number of pixels of the batch that take part (device)
};

__device__ __forceinline__ bool mask_tap(const LossMask& mk, int b, int y, int x, int H, int W) {
    if ((unsigned)b >= (unsigned)mk.Bm || (unsigned)x >= (unsigned)W || (unsigned)y >= (unsigned)H) return true;
    int xs = x, ys = y;
    if (mk.Wm != W || mk.Hm != H) {
        const float u = ((float)x + 0.5f) * (float)mk.Wm / (float)W - 0.5f;
        const float v = ((float)y + 0.5f) * (float)mk.Hm / (float)H - 0.5f;
        xs = max(0, min(mk.Wm - 1, (int)floorf(u + 0.5f)));
        ys = max(0, min(mk.Hm - 1, (int)floorf(v + 0.5f)));
    }
    return mk.mask[((size_t)b * mk.Hm + ys) * mk.Wm + xs] != 0;
}

// MAP_MODE (SsimLossMapMode, src/kernels/loss/PerPixelLoss.cuh:129-134): 0 no map; otherwise
// loss_map[pixel] += map_weight * (1 - mean over channels of v) with v = the SSIM (1), its
// contrast-structure factor D/B (2) or the structure term D / (2 sqrt(sigma1^2 sigma2^2) + C2) (3)
// (src/kernels/loss/FusedSSIM.cu:861-886,1009-1016).  MAP_MODE 4 is mode 1 plus the pixel's own weighted L1 term
// (DensifyLossMapMode::LossFull, src/kernels/loss/PerPixelLoss.cu:200-217,1127-1131).
//
// MASKED (per_pixel_losses.slang:161-176,290-291,365-375; FusedSSIM.cu:717-724,829-848,858-887,902-915,988-994):
// masked pixels add nothing to the L1 sum, which is divided by the number of unmasked pixels; masked samples are
// dropped from the SSIM window sums and the sums divided by the window's coverage; a window centred on a masked
// pixel scores 1 and sends no gradient; a masked pixel receives no gradient and maps to a perfect match.
template <int MAP_MODE, bool MASKED>
__global__ void __launch_bounds__(kLossThreads) loss_l1_ssim_kernel(
    const float* __restrict__ render, const float* __restrict__ gt, int B, int H, int W,
    float w_l1, float w_ssim, float* __restrict__ v_render, float* __restrict__ losses,
    float map_weight, float* __restrict__ loss_map, LossMask mk) {
    constexpr int NM = MASKED ? 6 : 5;  // moments per window
    extern __shared__ float smem[];
    float* sX = smem;
    float* sY = smem + kIn * kIn;
    float* sM = smem + kSmemA;          // [NM][kIn rows][kMStride]
    float* sD = smem;                   // [3][kMid][kDStride]   (aliases sX/sY)
    float* sH = smem + kSmemA;          // [3][kMid rows][kHStride] (aliases sM)
    float* sK = smem + kSmemA + kSmemBMasked;   // MASKED: [kIn][kIn] 1 = takes part
    __shared__ float red[2][kLossThreads / 32];

    const int b = blockIdx.z;
    const int ty0 = blockIdx.y * kLossTile, tx0 = blockIdx.x * kLossTile;
    const int64_t P = (int64_t)H * W;
    const float* R = render + (int64_t)b * P * 3;
    const float* G = gt + (int64_t)b * P * 3;
    float* V = v_render + (int64_t)b * P * 3;
    const float inv_n = 1.0f / (3.0f * (float)B * (float)W * (float)H);
    const float grad = -w_ssim * inv_n;
    const float n_l1 = MASKED ? (float)*mk.total : (float)B * (float)P;   // pixels the L1 mean is over
    const float l1_scale = w_l1 * (1.0f / 3.0f) / fmaxf(n_l1, 1.0f);
    const float kC1 = 0.01f * 0.01f, kC2 = 0.03f * 0.03f;
    float ssim_acc = 0.f, l1_acc = 0.f;

    for (int ch = 0; ch < 3; ++ch) {
        __syncthreads();
        // 1) input patch, zero padded
        for (int o = threadIdx.x; o < kIn * kIn; o += kLossThreads) {
            int ly = o / kIn, lx = o - ly * kIn;
            int gy = ty0 - 2 * kHalo + ly, gx = tx0 - 2 * kHalo + lx;
            float x = 0.f, y = 0.f;
            bool take = true;
            if (MASKED) {   // the mask patch is built with the first channel and kept
                if (ch == 0) {
                    take = mask_tap(mk, b, gy, gx, H, W);
                    sK[o] = take ? 1.f : 0.f;
                } else {
                    take = sK[o] != 0.f;
                }
            }
            if (take && (unsigned)gy < (unsigned)H && (unsigned)gx < (unsigned)W) {
                int64_t q = ((int64_t)gy * W + gx) * 3 + ch;
                x = R[q]; y = G[q];
            }
            sX[o] = x; sY[o] = y;
        }
        __syncthreads();
        // 2) row convolution of the five moments: rows 0..51, centre columns 5..46.
        //    One work item = 3 neighbouring outputs of a row: 13 + 13 shared-memory reads feed
        //    15 sums (instead of 22 reads per output).
        for (int o = threadIdx.x; o < kIn * (kMid / 3); o += kLossThreads) {
            const int ly = o / (kMid / 3), lc = (o - ly * (kMid / 3)) * 3;
            const float* xr = sX + ly * kIn + lc;
            const float* yr = sY + ly * kIn + lc;
            const float* kr = sK + ly * kIn + lc;
            float acc[3][NM];
#pragma unroll
            for (int q = 0; q < 3; ++q)
#pragma unroll
                for (int k = 0; k < NM; ++k) acc[q][k] = 0.f;
#pragma unroll
            for (int d = 0; d < 13; ++d) {
                const float x = xr[d], y = yr[d];
                const float xx = x * x, yy = y * y, xy = x * y;
                const float kk = MASKED ? kr[d] : 0.f;
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    const int tap = d - q;
                    if (tap >= 0 && tap < 11) {
                        const float wgt = cGaussW[tap];
                        acc[q][0] += x * wgt; acc[q][1] += xx * wgt; acc[q][2] += y * wgt; acc[q][3] += yy * wgt; acc[q][4] += xy * wgt;
                        if (MASKED) acc[q][NM - 1] += kk * wgt;
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 3; ++q)
#pragma unroll
                for (int k = 0; k < NM; ++k) sM[k * kIn * kMStride + ly * kMStride + lc + q] = acc[q][k];
        }
        __syncthreads();
        // 3) column convolution -> SSIM and its partials at the 42x42 window centres;
        //    one work item = 3 vertically neighbouring centres of a column.
        for (int o = threadIdx.x; o < (kMid / 3) * kMid; o += kLossThreads) {
            const int rg = o / kMid, c = o - rg * kMid;
            const int r0 = rg * 3;
            float m[3][NM];
#pragma unroll
            for (int q = 0; q < 3; ++q)
#pragma unroll
                for (int k = 0; k < NM; ++k) m[q][k] = 0.f;
#pragma unroll
            for (int k = 0; k < NM; ++k) {
                const float* col = sM + k * kIn * kMStride + r0 * kMStride + c;
#pragma unroll
                for (int d = 0; d < 13; ++d) {
                    const float v = col[d * kMStride];
#pragma unroll
                    for (int q = 0; q < 3; ++q) {
                        const int tap = d - q;
                        if (tap >= 0 && tap < 11) m[q][k] += v * cGaussW[tap];
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const int r = r0 + q;
                const int gy = ty0 - kHalo + r, gx = tx0 - kHalo + c;
                float d0 = 0.f, d1 = 0.f, d2 = 0.f;
                if ((unsigned)gy < (unsigned)H && (unsigned)gx < (unsigned)W) {
                    float inv_cov = 1.f;
                    bool centre = true;   // the window's centre pixel takes part
                    if (MASKED) {
                        inv_cov = 1.0f / fmaxf(m[q][NM - 1], 1e-6f);
                        centre = sK[(r + kHalo) * kIn + c + kHalo] != 0.f;
#pragma unroll
                        for (int k = 0; k < 5; ++k) m[q][k] *= inv_cov;
                    }
                    const float mu1 = m[q][0], mu2 = m[q][2];
                    const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
                    const float sigma1_sq = m[q][1] - mu1_sq, sigma2_sq = m[q][3] - mu2_sq, sigma12 = m[q][4] - mu1 * mu2;
                    const float A = mu1_sq + mu2_sq + kC1;
                    const float Bv = sigma1_sq + sigma2_sq + kC2;
                    const float C_ = 2.f * mu1 * mu2 + kC1;
                    const float D_ = 2.f * sigma12 + kC2;
                    // approximate reciprocals (two units in the last place), the arithmetic the reference's fast-math build has here
                    const float rA = __fdividef(1.0f, A), rB = __fdividef(1.0f, Bv);
                    const float rAB = rA * rB;
                    if (r >= kHalo && r < kHalo + kLossTile && c >= kHalo && c < kHalo + kLossTile) {
                        ssim_acc += centre ? (C_ * D_) * rAB : 1.0f;
                        if (MAP_MODE) {
                            float lm;
                            if (MAP_MODE == 2) lm = D_ / Bv;
                            else if (MAP_MODE == 3) lm = D_ / (2.f * sqrtf(fmaxf(sigma1_sq, 0.0f) * fmaxf(sigma2_sq, 0.0f)) + kC2);
                            else lm = (C_ * D_) * rAB;
                            if (!centre) lm = 1.0f;
                            // map += w * (1 - (v0 + v1 + v2) / 3) is linear in the channels' values, so each channel adds
                            // its share; the same thread meets this pixel in all three channels (no race)
                            float* slot = loss_map + (int64_t)b * P + (int64_t)gy * W + gx;
                            *slot += (ch == 0 ? map_weight : 0.f) - map_weight * (1.0f / 3.0f) * lm;
                        }
                    }
                    // each moment was divided by the coverage, so its reverse carries the same factor
                    const float gr = MASKED ? (centre ? grad * inv_cov : 0.f) : grad;
                    d0 = ((mu2 * 2.f * D_) * rAB - (mu2 * 2.f * C_) * rAB - (mu1 * 2.f * C_ * D_) * rAB * rA + (mu1 * 2.f * C_ * D_) * rAB * rB) * gr;
                    d1 = (-C_ * D_) * rAB * rB * gr;
                    d2 = (2.f * C_) * rAB * gr;
                }
                // sD aliases the input patches, which step 2 finished reading
                const int oo = r * kDStride + c;
                sD[oo] = d0; sD[kMid * kDStride + oo] = d1; sD[2 * kMid * kDStride + oo] = d2;
            }
        }
        __syncthreads();
        // 4) row convolution of the three partial maps: rows 0..41, centre columns 5..36;
        //    one work item = 2 neighbouring outputs of a row.
        for (int o = threadIdx.x; o < kMid * (kLossTile / 2); o += kLossThreads) {
            const int r = o / (kLossTile / 2), c = (o - r * (kLossTile / 2)) * 2;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float* row = sD + k * kMid * kDStride + r * kDStride + c;
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int d = 0; d < 12; ++d) {
                    const float v = row[d];
                    if (d < 11) s0 += v * cGaussW[d];
                    if (d >= 1) s1 += v * cGaussW[d - 1];
                }
                sH[k * kMid * kHStride + r * kHStride + c] = s0;
                sH[k * kMid * kHStride + r * kHStride + c + 1] = s1;
            }
        }
        __syncthreads();
        // 5) column convolution and the gradient of this channel; one work item = 4
        //    vertically neighbouring pixels of a column (256 items = one per thread).
        for (int o = threadIdx.x; o < (kLossTile / 4) * kLossTile; o += kLossThreads) {
            const int rg = o / kLossTile, c = o - rg * kLossTile;
            const int r0 = rg * 4;
            float sacc[4][3];
#pragma unroll
            for (int q = 0; q < 4; ++q) sacc[q][0] = sacc[q][1] = sacc[q][2] = 0.f;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float* col = sH + k * kMid * kHStride + r0 * kHStride + c;
#pragma unroll
                for (int d = 0; d < 14; ++d) {
                    const float v = col[d * kHStride];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int tap = d - q;
                        if (tap >= 0 && tap < 11) sacc[q][k] += v * cGaussW[tap];
                    }
                }
            }
            const int gx = tx0 + c;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int gy = ty0 + r0 + q;
                if (gy < H && gx < W) {
                    const int64_t qi = ((int64_t)gy * W + gx) * 3 + ch;
                    const float p1 = R[qi], p2 = G[qi];
                    const float diff = p1 - p2;
                    const bool take = !MASKED || sK[(r0 + q + 2 * kHalo) * kIn + c + 2 * kHalo] != 0.f;
                    const float sg = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
                    if (take) {
                        l1_acc += fabsf(diff);
                        V[qi] = l1_scale * sg + (sacc[q][0] + (2.f * p1) * sacc[q][1] + p2 * sacc[q][2]);
                        // |w_l1 * (|d0| + |d1| + |d2|) / 3|, one channel's share at a time (this thread owns the pixel in stage 5)
                        if (MAP_MODE == 4) loss_map[(int64_t)b * P + (int64_t)gy * W + gx] += fabsf(w_l1) * (1.0f / 3.0f) * fabsf(diff);
                    } else {
                        V[qi] = 0.f;
                    }
                }
            }
        }
    }
    // block reduction of the two scalars
    ssim_acc = warp_sum(ssim_acc);
    l1_acc = warp_sum(l1_acc);
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = ssim_acc; red[1][threadIdx.x >> 5] = l1_acc; }
    __syncthreads();
    if (threadIdx.x == 0 && losses) {
        float s = 0.f, l = 0.f;
        for (int k = 0; k < kLossThreads / 32; ++k) { s += red[0][k]; l += red[1][k]; }
        float l1_mean = MASKED ? l * (1.0f / 3.0f) / fmaxf(n_l1, 1.0f) : l * inv_n, ssim_mean = s * inv_n;
        atomicAdd(&losses[0], l1_mean);
        atomicAdd(&losses[1], ssim_mean);
        float tot = w_l1 * l1_mean - w_ssim * ssim_mean;
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) tot += w_ssim;
        atomicAdd(&losses[2], tot);
    }
}

template <int MAP_MODE, bool MASKED>
static int launch_loss_mode(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                            float* d_v_render, float* d_losses, float map_weight, float* d_loss_map, const LossMask& mk, cudaStream_t st) {
    constexpr int smem = MASKED ? kLossSmemBytesMasked : kLossSmemBytes;
    if (int e = ensure_dynamic_smem((const void*)loss_l1_ssim_kernel<MAP_MODE, MASKED>, smem)) return e;
    dim3 grid((unsigned)ceil_div(W, kLossTile), (unsigned)ceil_div(H, kLossTile), (unsigned)B);
    loss_l1_ssim_kernel<MAP_MODE, MASKED><<<grid, kLossThreads, smem, st>>>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses,
                                                                            map_weight, d_loss_map, mk);
    SSB_LAUNCHED("loss_l1_ssim_kernel");
    return SSB_OK;
}

int launch_loss(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                float* d_v_render, float* d_losses, cudaStream_t st) {
    return launch_loss_mode<0, false>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, 0.f, nullptr, LossMask{}, st);
}

// d_losses is added to (not cleared).  map_mode 0..3 = SsimLossMapMode, 4 = full SSIM plus the per-pixel L1 term;
// mk.mask == nullptr: no mask.
static int launch_loss_any(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim, float* d_v_render,
                           float* d_losses, int map_mode, float map_weight, float* d_loss_map, const LossMask& mk, cudaStream_t st) {
#define SSB_LOSS_CASE(MODE)                                                                                                              \
    case MODE:                                                                                                                           \
        return mk.mask ? launch_loss_mode<MODE, true>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, map_weight, d_loss_map, mk, st) \
                       : launch_loss_mode<MODE, false>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, map_weight, d_loss_map, mk, st);
    switch (map_mode) {
        SSB_LOSS_CASE(1)
        SSB_LOSS_CASE(2)
        SSB_LOSS_CASE(3)
        SSB_LOSS_CASE(4)
        default:
            return mk.mask ? launch_loss_mode<0, true>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, 0.f, nullptr, mk, st)
                           : launch_loss_mode<0, false>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, 0.f, nullptr, mk, st);
    }
#undef SSB_LOSS_CASE
}

int launch_loss_map(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                    float* d_v_render, float* d_losses, int map_mode, float map_weight, float* d_loss_map, cudaStream_t st) {
    return launch_loss_any(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, map_mode, map_weight, d_loss_map, LossMask{}, st);
}

// ---- multi-scale loss -------------------------------------------------------------------------------------------
// compute_multi_scale_per_pixel_losses (src/kernels/loss/PerPixelLoss.cu:941-1363) for the colour modalities.

// Number of pixels of an [B][H][W] image that take part under a mask of its own or another size.
__global__ void mask_count_kernel(LossMask mk, int B, int H, int W, unsigned long long* __restrict__ total) {
    const int64_t n = (int64_t)B * H * W;
    unsigned cnt = 0;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % W), y = (int)((i / W) % H), b = (int)(i / ((int64_t)W * H));
        cnt += mask_tap(mk, b, y, x, H, W);
    }
    cnt = __reduce_add_sync(0xffffffffu, cnt);
    if ((threadIdx.x & 31) == 0 && cnt) atomicAdd(total, (unsigned long long)cnt);
}

// One pyramid level from the previous one: render and target pool 2x2 (the mean over the children that take part when
// the mask has the image's size, the plain mean when none does or there is no such mask; avg_pool_downsample_float_kernel
// :617-637 and avg_pool_downsample_masked_float_kernel :675-701).
template <bool MASK_SAME>
__global__ void pool_images_kernel(const float* __restrict__ r_hi, const float* __restrict__ g_hi, const uint8_t* __restrict__ m_hi,
                                   int B, int Hh, int Wh, int Hl, int Wl, float* __restrict__ r_lo, float* __restrict__ g_lo) {
    const int64_t n = (int64_t)B * Hl * Wl;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % Wl), y = (int)((i / Wl) % Hl), b = (int)(i / ((int64_t)Wl * Hl));
        float acc[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, box[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        int cnt = 0;
#pragma unroll
        for (int dy = 0; dy < 2; ++dy)
#pragma unroll
            for (int dx = 0; dx < 2; ++dx) {
                const int64_t q = ((int64_t)b * Hh + min(2 * y + dy, Hh - 1)) * Wh + min(2 * x + dx, Wh - 1);
                const bool valid = MASK_SAME && m_hi[q] != 0;
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    const float rv = r_hi[3 * q + c], gv = g_hi[3 * q + c];
                    box[c] += rv; box[3 + c] += gv;
                    if (valid) { acc[c] += rv; acc[3 + c] += gv; }
                }
                cnt += valid;
            }
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            r_lo[3 * i + c] = cnt ? acc[c] / (float)cnt : 0.25f * box[c];
            g_lo[3 * i + c] = cnt ? acc[3 + c] / (float)cnt : 0.25f * box[3 + c];
        }
    }
}

// The mask halves its own size: a coarse pixel takes part when at least two of its four children do
// (avg_pool_downsample_bool_kernel, :723-740).
__global__ void pool_mask_kernel(const uint8_t* __restrict__ m_hi, int B, int Hh, int Wh, int Hl, int Wl, uint8_t* __restrict__ m_lo) {
    const int64_t n = (int64_t)B * Hl * Wl;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % Wl), y = (int)((i / Wl) % Hl), b = (int)(i / ((int64_t)Wl * Hl));
        int v = 0;
#pragma unroll
        for (int dy = 0; dy < 2; ++dy)
#pragma unroll
            for (int dx = 0; dx < 2; ++dx) v += m_hi[((int64_t)b * Hh + min(2 * y + dy, Hh - 1)) * Wh + min(2 * x + dx, Wh - 1)] != 0;
        m_lo[i] = v >= 2;
    }
}

struct FoldLevels {
    int n;                       // coarse levels (1..3)
    const float* v[3];           // their gradients [B][Hs][Ws][3]
    const float* lm[3];          // their loss maps [B][Hs][Ws] (or nullptr)
    int H[3], W[3];
};

// All coarse levels folded into the full-resolution gradient and loss map in one pass:
// v = (v_0 + sum_s 0.25^s v_s[y >> s][x >> s]) / S (0 where the mask of the image's size says "masked"),
// map = (map_0 + sum_s map_s[y >> s][x >> s]) / S; a coarse pixel that does not exist adds nothing
// (avg_pool_upsample_float_kernel :926-943 applied level by level, :1262-1336).
__global__ void fold_levels_kernel(FoldLevels f, int B, int H, int W, const uint8_t* __restrict__ mask_same, float* __restrict__ v0,
                                   float* __restrict__ map0) {
    const int64_t n = (int64_t)B * H * W;
    const float inv_s = 1.0f / (float)(f.n + 1);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % W), y = (int)((i / W) % H), b = (int)(i / ((int64_t)W * H));
        float g0 = v0[3 * i], g1 = v0[3 * i + 1], g2 = v0[3 * i + 2];
        float m = map0 ? map0[i] : 0.f;
        float wgt = 1.f;
        for (int s = 0; s < f.n; ++s) {
            wgt *= 0.25f;
            const int ys = y >> (s + 1), xs = x >> (s + 1);
            if (ys >= f.H[s] || xs >= f.W[s]) continue;
            const int64_t q = ((int64_t)b * f.H[s] + ys) * f.W[s] + xs;
            g0 += wgt * f.v[s][3 * q]; g1 += wgt * f.v[s][3 * q + 1]; g2 += wgt * f.v[s][3 * q + 2];
            if (map0) m += f.lm[s][q];
        }
        const float keep = (mask_same && !mask_same[i]) ? 0.f : inv_s;
        v0[3 * i] = g0 * keep; v0[3 * i + 1] = g1 * keep; v0[3 * i + 2] = g2 * keep;
        if (map0) map0[i] = m * inv_s;
    }
}

// losses[0] += mean over levels of the L1 term, [1] += level 0's SSIM, [2] += mean over levels of the total
__global__ void fold_losses_kernel(const float* __restrict__ level_losses, int n_levels, float* __restrict__ losses) {
    float l1 = 0.f, tot = 0.f;
    for (int s = 0; s < n_levels; ++s) { l1 += level_losses[3 * s]; tot += level_losses[3 * s + 2]; }
    losses[0] += l1 / (float)n_levels;
    losses[1] += level_losses[1];
    losses[2] += tot / (float)n_levels;
}

static inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

struct LossLevels {
    int n, H[4], W[4], Hm[4], Wm[4];
    int64_t off_r[4], off_g[4], off_v[4], off_lm[4], off_m[4], off_counts, off_losses, bytes;
};

static LossLevels plan_levels(int B, int H, int W, int n_scales, bool masked, int Hm, int Wm, bool want_map) {
    LossLevels L{};
    L.n = n_scales;
    int64_t off = 0;
    auto take = [&](int64_t bytes) { int64_t o = off; off += align256(bytes); return o; };
    L.off_counts = take(4 * sizeof(unsigned long long));
    L.off_losses = take(4 * 3 * sizeof(float));
    for (int s = 0; s < n_scales; ++s) {
        L.H[s] = s ? std::max(1, L.H[s - 1] / 2) : H;
        L.W[s] = s ? std::max(1, L.W[s - 1] / 2) : W;
        L.Hm[s] = masked ? (s ? std::max(1, L.Hm[s - 1] / 2) : Hm) : 0;
        L.Wm[s] = masked ? (s ? std::max(1, L.Wm[s - 1] / 2) : Wm) : 0;
        if (s == 0) continue;
        const int64_t px = (int64_t)B * L.H[s] * L.W[s];
        L.off_r[s] = take(px * 12);
        L.off_g[s] = take(px * 12);
        L.off_v[s] = take(px * 12);
        L.off_lm[s] = want_map ? take(px * 4) : 0;
        L.off_m[s] = masked ? take((int64_t)B * L.Hm[s] * L.Wm[s]) : 0;
    }
    L.bytes = off;
    return L;
}

int64_t loss_workspace_bytes(int B, int H, int W, const SsbLossConfig& cfg) {
    return plan_levels(B, H, W, cfg.num_scales, cfg.d_mask != nullptr, cfg.mask_h, cfg.mask_w, cfg.loss_map_mode != 0).bytes;
}

// d_losses is added to (not cleared); the caller has validated cfg.
int launch_loss_multi(const float* d_render, const float* d_gt, int B, int H, int W, const SsbLossConfig& cfg, float* d_v_render,
                      float* d_losses, float* d_loss_map, void* d_ws, int64_t ws_bytes, cudaStream_t st) {
    const bool masked = cfg.d_mask != nullptr;
    const bool want_map = cfg.loss_map_mode != 0 && d_loss_map;
    const LossLevels L = plan_levels(B, H, W, cfg.num_scales, masked, cfg.mask_h, cfg.mask_w, cfg.loss_map_mode != 0);
    if (ws_bytes < L.bytes || !d_ws) {
        set_error("ssb_loss_multi_scale: workspace of %lld bytes, %lld needed", (long long)ws_bytes, (long long)L.bytes);
        return SSB_ERR_CAPACITY;
    }
    char* ws = (char*)d_ws;
    unsigned long long* counts = (unsigned long long*)(ws + L.off_counts);
    float* level_losses = (float*)(ws + L.off_losses);
    SSB_CUDA(cudaMemsetAsync(ws, 0, (size_t)(L.off_losses + 4 * 3 * sizeof(float)), st));   // counts and per-level losses
    const int threads = 256;
    auto blocks = [&](int64_t n) { return (unsigned)std::min<int64_t>(ceil_div(std::max<int64_t>(n, 1), threads), 148 * 8); };
    const float* r[4] = {d_render}; const float* g[4] = {d_gt}; const uint8_t* m[4] = {cfg.d_mask};
    float* v[4] = {d_v_render}; float* lm[4] = {want_map ? d_loss_map : nullptr};
    for (int s = 1; s < L.n; ++s) {
        r[s] = (float*)(ws + L.off_r[s]); g[s] = (float*)(ws + L.off_g[s]); v[s] = (float*)(ws + L.off_v[s]);
        lm[s] = want_map ? (float*)(ws + L.off_lm[s]) : nullptr;
        m[s] = masked ? (uint8_t*)(ws + L.off_m[s]) : nullptr;
        const int64_t px = (int64_t)B * L.H[s] * L.W[s];
        const bool same = masked && L.Hm[s - 1] == L.H[s - 1] && L.Wm[s - 1] == L.W[s - 1];
        if (same)
            pool_images_kernel<true><<<blocks(px), threads, 0, st>>>(r[s - 1], g[s - 1], m[s - 1], B, L.H[s - 1], L.W[s - 1], L.H[s], L.W[s],
                                                                   (float*)r[s], (float*)g[s]);
        else
            pool_images_kernel<false><<<blocks(px), threads, 0, st>>>(r[s - 1], g[s - 1], nullptr, B, L.H[s - 1], L.W[s - 1], L.H[s], L.W[s],
                                                                    (float*)r[s], (float*)g[s]);
        SSB_LAUNCHED("pool_images_kernel");
        if (masked) {
            pool_mask_kernel<<<blocks((int64_t)B * L.Hm[s] * L.Wm[s]), threads, 0, st>>>(m[s - 1], B, L.Hm[s - 1], L.Wm[s - 1], L.Hm[s], L.Wm[s],
                                                                                      (uint8_t*)m[s]);
            SSB_LAUNCHED("pool_mask_kernel");
        }
    }
    // SsimLossMapMode of the kernel for each DensifyLossMapMode: LossFull -> full SSIM + the pixel's L1 term
    const int kernel_mode = !want_map ? 0 : (cfg.loss_map_mode == 1 ? 4 : cfg.loss_map_mode - 1);
    for (int s = 0; s < L.n; ++s) {
        LossMask mk{m[s], B, L.Hm[s], L.Wm[s], counts + s};
        const int64_t px = (int64_t)B * L.H[s] * L.W[s];
        if (masked) {
            mask_count_kernel<<<blocks(px), threads, 0, st>>>(mk, B, L.H[s], L.W[s], counts + s);
            SSB_LAUNCHED("mask_count_kernel");
        }
        if (lm[s]) SSB_CUDA(cudaMemsetAsync(lm[s], 0, (size_t)px * sizeof(float), st));
        float* dst = L.n == 1 ? d_losses : level_losses + 3 * s;
        if (int e = launch_loss_any(r[s], g[s], B, L.H[s], L.W[s], cfg.w_l1, cfg.w_ssim, v[s], dst, kernel_mode, cfg.w_ssim, lm[s], mk, st)) return e;
    }
    if (L.n > 1) {
        FoldLevels f{};
        f.n = L.n - 1;
        for (int s = 1; s < L.n; ++s) { f.v[s - 1] = v[s]; f.lm[s - 1] = lm[s]; f.H[s - 1] = L.H[s]; f.W[s - 1] = L.W[s]; }
        const bool same0 = masked && cfg.mask_h == H && cfg.mask_w == W;
        fold_levels_kernel<<<blocks((int64_t)B * H * W), threads, 0, st>>>(f, B, H, W, same0 ? cfg.d_mask : nullptr, d_v_render, lm[0]);
        SSB_LAUNCHED("fold_levels_kernel");
        if (d_losses) {
            fold_losses_kernel<<<1, 1, 0, st>>>(level_losses, L.n, d_losses);
            SSB_LAUNCHED("fold_losses_kernel");
        }
    }
    return SSB_OK;
}

int check_loss_config(const SsbLossConfig* cfg, const char* who) {
    SSB_REQUIRE(cfg, "%s: NULL config", who);
    SSB_REQUIRE(cfg->num_scales >= 1 && cfg->num_scales <= 4, "%s: num_scales %d is not in 1..4", who, cfg->num_scales);
    SSB_REQUIRE(cfg->loss_map_mode >= 0 && cfg->loss_map_mode <= 10, "%s: loss_map_mode %d is not a DensifyLossMapMode", who, cfg->loss_map_mode);
    if (cfg->loss_map_mode > 4) {
        set_error("%s: loss_map_mode %d (edge-aware and non-maximum-suppression maps) is not built", who, cfg->loss_map_mode);
        return SSB_ERR_UNSUPPORTED;
    }
    SSB_REQUIRE(!cfg->d_mask || (cfg->mask_h > 0 && cfg->mask_w > 0), "%s: mask without a size", who);
    return SSB_OK;
}

}  // namespace ssb

extern "C" int ssb_loss_l1_ssim_fwdbwd(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                                       float w_l1, float w_ssim, float* d_v_render, float* d_losses, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_render && d_gt && d_v_render, "ssb_loss_l1_ssim_fwdbwd: NULL argument");
    SSB_REQUIRE(n_images >= 0 && height > 0 && width > 0, "ssb_loss_l1_ssim_fwdbwd: bad sizes");
    if (n_images == 0) return SSB_OK;
    if (d_losses) SSB_CUDA(cudaMemsetAsync(d_losses, 0, 3 * sizeof(float), (cudaStream_t)stream));
    return launch_loss(d_render, d_gt, n_images, height, width, w_l1, w_ssim, d_v_render, d_losses, (cudaStream_t)stream);
}

extern "C" int ssb_loss_l1_ssim_fwdbwd_map(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                                           float w_l1, float w_ssim, float* d_v_render, float* d_losses,
                                           int32_t ssim_loss_map_mode, float ssim_loss_map_weight, float* d_loss_map, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_render && d_gt && d_v_render, "ssb_loss_l1_ssim_fwdbwd_map: NULL argument");
    SSB_REQUIRE(n_images >= 0 && height > 0 && width > 0, "ssb_loss_l1_ssim_fwdbwd_map: bad sizes");
    SSB_REQUIRE(ssim_loss_map_mode >= 0 && ssim_loss_map_mode <= 3, "ssb_loss_l1_ssim_fwdbwd_map: mode %d is not a SsimLossMapMode", ssim_loss_map_mode);
    SSB_REQUIRE(ssim_loss_map_mode == 0 || d_loss_map, "ssb_loss_l1_ssim_fwdbwd_map: d_loss_map is NULL");
    if (n_images == 0) return SSB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (d_losses) SSB_CUDA(cudaMemsetAsync(d_losses, 0, 3 * sizeof(float), st));
    return launch_loss_map(d_render, d_gt, n_images, height, width, w_l1, w_ssim, d_v_render, d_losses, ssim_loss_map_mode, ssim_loss_map_weight,
                           d_loss_map, st);
}

extern "C" int64_t ssb_loss_workspace_bytes(int32_t n_images, int32_t height, int32_t width, const SsbLossConfig* cfg) {
    using namespace ssb;
    if (check_loss_config(cfg, "ssb_loss_workspace_bytes") || n_images < 0 || height <= 0 || width <= 0) return SSB_ERR_INVALID_ARGUMENT;
    return loss_workspace_bytes(n_images, height, width, *cfg);
}

extern "C" int ssb_loss_multi_scale(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                                    const SsbLossConfig* cfg, float* d_v_render, float* d_losses, float* d_loss_map, void* d_workspace,
                                    int64_t workspace_bytes, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_render && d_gt && d_v_render, "ssb_loss_multi_scale: NULL argument");
    SSB_REQUIRE(n_images >= 0 && height > 0 && width > 0, "ssb_loss_multi_scale: bad sizes");
    if (int e = check_loss_config(cfg, "ssb_loss_multi_scale")) return e;
    SSB_REQUIRE(cfg->loss_map_mode == 0 || d_loss_map, "ssb_loss_multi_scale: d_loss_map is NULL");
    if (n_images == 0) return SSB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (d_losses) SSB_CUDA(cudaMemsetAsync(d_losses, 0, 3 * sizeof(float), st));
    return launch_loss_multi(d_render, d_gt, n_images, height, width, *cfg, d_v_render, d_losses, d_loss_map, d_workspace, workspace_bytes, st);
}
