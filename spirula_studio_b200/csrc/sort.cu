// Stable least-significant-digit radix sort of (64-bit key, 32-bit value) pairs
// on a key bit range, 8 bits per pass.  Stands in for
// cub::DeviceRadixSort::SortPairs<int64,int32> as the reference calls it
// (src/kernels/tile/IntersectTile.cu:487-497; contract in
// src/backend/common/SortScan.h:53-56).
//
// The element count is read from device memory, so the sort can follow key
// generation without a host round trip.  Each pass is three launches over a
// fixed grid of kSortBlocks blocks, block b owning the contiguous slice
// [b*ipb, (b+1)*ipb) of the input:
//   1. digit histogram of every slice           -> hist[digit][block]
//   2. exclusive scan of hist in (digit, block) order
//   3. stable scatter: per 4096-key tile, keys are ranked inside their warp with
//      match.any (equal digits keep their order), warps are offset against each
//      other through a 8x256 shared table, and each key goes to
//      base[digit] + rank.
// No block ever waits on another block, so there is nothing that can spin.
#include "ssb_common.cuh"

namespace ssb {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortItems = 16;                                  // keys per thread per tile
constexpr int kSortTile = kSortThreads * kSortItems;            // 4096
constexpr int kSortWarpSpan = 32 * kSortItems;                  // 512 consecutive keys per warp
constexpr int kSortBlocks = 148 * 4;
constexpr int kRadix = 256;

__device__ __forceinline__ int64_t slice_len(int64_t n) {
    int64_t ipb = (n + kSortBlocks - 1) / kSortBlocks;
    return (ipb + kSortTile - 1) / kSortTile * kSortTile;
}

// Counts digits of one warp round into the warp's private table.
__device__ __forceinline__ int warp_rank(int* cnt_w, int digit, bool valid, int lane) {
    unsigned peers = __match_any_sync(0xffffffffu, valid ? digit : (kRadix + lane));
    int rank = __popc(peers & ((1u << lane) - 1u));
    int leader = __ffs(peers) - 1;
    int prev = 0;
    if (lane == leader && valid) {
        prev = cnt_w[digit];
        cnt_w[digit] = prev + __popc(peers);
    }
    prev = __shfl_sync(0xffffffffu, prev, leader);
    __syncwarp();
    return prev + rank;
}

__global__ void __launch_bounds__(kSortThreads) sort_hist_kernel(
    const uint64_t* __restrict__ keys, const int64_t* __restrict__ n_ptr, int64_t capacity, int shift, int mask,
    int32_t* __restrict__ hist) {
    __shared__ int cnt[kSortWarps][kRadix];
    const int64_t n = min(*n_ptr, capacity);
    const int64_t ipb = slice_len(n);
    const int64_t begin = (int64_t)blockIdx.x * ipb;
    const int64_t end = min(n, begin + ipb);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&cnt[0][0])[i] = 0;
    __syncthreads();
    for (int64_t tile = begin; tile < end; tile += kSortTile) {
        int64_t wbase = tile + (int64_t)w * kSortWarpSpan;
#pragma unroll 4
        for (int r = 0; r < kSortItems; ++r) {
            int64_t i = wbase + r * 32 + lane;
            bool valid = i < end;
            int d = valid ? (int)((keys[i] >> shift) & (uint64_t)mask) : 0;
            warp_rank(cnt[w], d, valid, lane);
        }
    }
    __syncthreads();
    int d = threadIdx.x;
    int s = 0;
#pragma unroll
    for (int k = 0; k < kSortWarps; ++k) s += cnt[k][d];
    hist[d * kSortBlocks + blockIdx.x] = s;
}

__global__ void __launch_bounds__(1024) sort_scan_kernel(int32_t* __restrict__ hist) {
    constexpr int total = kRadix * kSortBlocks;
    constexpr int per = (total + 1023) / 1024;
    __shared__ int warp_tot[32];
    int begin = threadIdx.x * per, end = min(total, begin + per);
    int s = 0;
    for (int i = begin; i < end; ++i) s += hist[i];
    int inc = s;
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if ((threadIdx.x & 31) >= o) inc += t;
    }
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    if (threadIdx.x < 32) {
        int wv = warp_tot[threadIdx.x], winc = wv;
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (threadIdx.x >= o) winc += t;
        }
        warp_tot[threadIdx.x] = winc - wv;
    }
    __syncthreads();
    int run = warp_tot[threadIdx.x >> 5] + inc - s;
    for (int i = begin; i < end; ++i) { int v = hist[i]; hist[i] = run; run += v; }
}

__global__ void __launch_bounds__(kSortThreads) sort_scatter_kernel(
    const uint64_t* __restrict__ keys_in, const int32_t* __restrict__ vals_in,
    uint64_t* __restrict__ keys_out, int32_t* __restrict__ vals_out,
    const int64_t* __restrict__ n_ptr, int64_t capacity, int shift, int mask, const int32_t* __restrict__ hist) {
    __shared__ int cnt[kSortWarps][kRadix];
    __shared__ int base[kRadix];
    const int64_t n = min(*n_ptr, capacity);
    const int64_t ipb = slice_len(n);
    const int64_t begin = (int64_t)blockIdx.x * ipb;
    const int64_t end = min(n, begin + ipb);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    base[threadIdx.x] = hist[threadIdx.x * kSortBlocks + blockIdx.x];
    for (int64_t tile = begin; tile < end; tile += kSortTile) {
        for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&cnt[0][0])[i] = 0;
        __syncthreads();
        int64_t wbase = tile + (int64_t)w * kSortWarpSpan;
        uint64_t key[kSortItems];
        int rank[kSortItems];
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            int64_t i = wbase + r * 32 + lane;
            key[r] = i < end ? keys_in[i] : 0;
        }
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            int64_t i = wbase + r * 32 + lane;
            bool valid = i < end;
            int d = (int)((key[r] >> shift) & (uint64_t)mask);
            rank[r] = warp_rank(cnt[w], d, valid, lane);
        }
        __syncthreads();
        {
            int d = threadIdx.x;
            int run = base[d];
#pragma unroll
            for (int k = 0; k < kSortWarps; ++k) { int t = cnt[k][d]; cnt[k][d] = run; run += t; }
            base[d] = run;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            int64_t i = wbase + r * 32 + lane;
            if (i < end) {
                int d = (int)((key[r] >> shift) & (uint64_t)mask);
                int64_t pos = (int64_t)cnt[w][d] + rank[r];
                keys_out[pos] = key[r];
                vals_out[pos] = vals_in[i];
            }
        }
        __syncthreads();
    }
}

}  // namespace ssb

extern "C" {

int64_t ssb_sort_workspace_bytes(int64_t capacity) {
    (void)capacity;
    return (int64_t)ssb::kRadix * ssb::kSortBlocks * 4;
}

int ssb_sort_pairs_u64(int64_t* d_keys_a, int32_t* d_vals_a, int64_t* d_keys_b, int32_t* d_vals_b,
                       const int64_t* d_n, int64_t capacity, int32_t begin_bit, int32_t end_bit,
                       void* d_workspace, int64_t workspace_bytes, int32_t* selector, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_keys_a && d_vals_a && d_keys_b && d_vals_b && d_n && d_workspace && selector, "ssb_sort_pairs_u64: NULL argument");
    SSB_REQUIRE(begin_bit >= 0 && end_bit <= 64 && begin_bit <= end_bit, "ssb_sort_pairs_u64: bad bit range [%d, %d)", begin_bit, end_bit);
    SSB_REQUIRE(capacity >= 0 && capacity < ((int64_t)1 << 31), "ssb_sort_pairs_u64: capacity must fit int32");
    SSB_REQUIRE(workspace_bytes >= ssb_sort_workspace_bytes(capacity), "ssb_sort_pairs_u64: workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    int32_t* hist = (int32_t*)d_workspace;
    int sel = 0;
    uint64_t* kbuf[2] = {(uint64_t*)d_keys_a, (uint64_t*)d_keys_b};
    int32_t* vbuf[2] = {d_vals_a, d_vals_b};
    for (int bit = begin_bit; bit < end_bit && capacity > 0; bit += 8) {
        int nbits = end_bit - bit < 8 ? end_bit - bit : 8;
        int mask = (1 << nbits) - 1;
        sort_hist_kernel<<<kSortBlocks, kSortThreads, 0, st>>>(kbuf[sel], d_n, capacity, bit, mask, hist);
        SSB_LAUNCHED("sort_hist_kernel");
        sort_scan_kernel<<<1, 1024, 0, st>>>(hist);
        SSB_LAUNCHED("sort_scan_kernel");
        sort_scatter_kernel<<<kSortBlocks, kSortThreads, 0, st>>>(kbuf[sel], vbuf[sel], kbuf[sel ^ 1], vbuf[sel ^ 1], d_n, capacity, bit, mask, hist);
        SSB_LAUNCHED("sort_scatter_kernel");
        sel ^= 1;
    }
    *selector = sel;
    return SSB_OK;
}

}  // extern "C"
