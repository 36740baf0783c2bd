// Stable least-significant-digit radix sort of (64-bit key, 32-bit value) pairs
// on a key bit range.  Stands in for cub::DeviceRadixSort::SortPairs<int64,int32>
// as the reference calls it (src/kernels/tile/IntersectTile.cu:487-497; contract
// in src/backend/common/SortScan.h:53-56).
//
// The element count is read from device memory, so the sort follows key
// generation without a host round trip.  Up to 9 bits are sorted per pass and
// each pass is ONE launch that reads and writes every pair once (24 B/pair):
//   * a 4096-pair tile is taken by ticket (atomic counter), so every tile with a
//     smaller index is already running or finished;
//   * keys are ranked inside their warp by matching digits with one ballot per
//     digit bit (equal digits keep their order), warps are offset against each
//     other through an 8 x 512 table in shared memory;
//   * the tile publishes its per-digit counts in a descriptor row and looks
//     back over its predecessors' rows, sixteen rows per step (count-only -> add
//     and go on; inclusive prefix -> add and stop), then publishes its own
//     inclusive prefix;
//   * the tile is staged in digit order in shared memory and written out in that
//     order, so neighbouring threads write neighbouring addresses;
//   * while the keys are in registers the tile also counts the NEXT pass's
//     digit, so the digit totals a pass needs were produced by the pass before
//     it (a small kernel produces them for the first pass).
// Every wait on a descriptor is bounded: after kSpinLimit polls the tile records
// an error, goes on with what it has and still publishes its row, so nothing
// can hang; the host reports the error on its next synchronising call.
#include "ssb_common.cuh"

namespace ssb {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortItems = 16;                                  // keys per thread per tile
constexpr int kSortTile = kSortThreads * kSortItems;            // 4096
constexpr int kSortWarpSpan = 32 * kSortItems;                  // 512 consecutive keys per warp
constexpr int kRadixBits = 9;
constexpr int kRadix = 1 << kRadixBits;                         // 512 digit values
constexpr int kMaxPasses = 8;
constexpr uint32_t kFlagAggregate = 1u << 30, kFlagInclusive = 2u << 30, kValueMask = (1u << 30) - 1u;
constexpr int kSpinLimit = 1 << 22;
constexpr int kLookWindow = 16;

struct SortHeader {                 // lives at the start of the workspace
    uint32_t hist[kMaxPasses][kRadix];
    uint32_t ticket[kMaxPasses];
    uint32_t error;
    uint32_t pad[7];
#ifdef SSB_SORT_PROFILE
    unsigned long long prof[8];
#endif
};

__device__ __forceinline__ int digit_of(uint64_t key, int shift, int mask) { return (int)((key >> shift) & (uint64_t)mask); }

// Lanes of the warp whose digit equals this lane's: nbits independent ballots and an AND
// chain (match.any serialises over the distinct values, which with 9-bit digits is
// nearly every lane).  Invalid lanes match nobody.
__device__ __forceinline__ unsigned match_digit(int digit, bool valid, int nbits) {
    unsigned peers = __ballot_sync(0xffffffffu, valid);
#pragma unroll
    for (int b = 0; b < kRadixBits; ++b) {
        if (b < nbits) {
            const bool bit = (digit >> b) & 1;
            const unsigned bal = __ballot_sync(0xffffffffu, bit);
            peers &= bit ? bal : ~bal;
        }
    }
    return valid ? peers : 0u;
}

// Rank of this lane's key among the lanes of the round with the same digit, plus
// the warp's running count of that digit; updates the running count.
__device__ __forceinline__ int warp_rank(int* cnt_w, int digit, bool valid, int lane, int nbits) {
    const unsigned peers = match_digit(digit, valid, nbits);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const int leader = __ffs(peers) - 1;
    int prev = 0;
    if (valid && lane == leader) {
        prev = cnt_w[digit];
        cnt_w[digit] = prev + __popc(peers);
    }
    prev = __shfl_sync(0xffffffffu, prev, leader < 0 ? 0 : leader);
    __syncwarp();
    return prev + rank;
}

// Adds this lane's digit to a block-wide table.  A plain shared-memory atomic per lane costs
// one instruction (the hardware serialises lanes that hit the same counter); matching the
// lanes first would cost some forty.
__device__ __forceinline__ void warp_count(int* table, int digit, bool valid) {
    if (valid) atomicAdd(&table[digit], 1);
}

// Digit totals of the first pass; also clears descriptor region 0 for the tiles in use.
__global__ void __launch_bounds__(kSortThreads) sort_first_hist_kernel(
    const uint64_t* __restrict__ keys, const int64_t* __restrict__ n_ptr, int64_t capacity, int shift, int mask,
    SortHeader* __restrict__ hdr, uint32_t* __restrict__ desc0) {
    __shared__ int table[kRadix];
    const int64_t n = min(*n_ptr, capacity);
    const int64_t n_tiles = (n + kSortTile - 1) / kSortTile;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < kRadix; i += kSortThreads) table[i] = 0;
    __syncthreads();
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        for (int i = threadIdx.x; i < kRadix; i += kSortThreads) desc0[tile * kRadix + i] = 0u;
        const int64_t wbase = tile * kSortTile + (int64_t)w * kSortWarpSpan;
#pragma unroll 4
        for (int r = 0; r < kSortItems; ++r) {
            int64_t i = wbase + r * 32 + lane;
            bool valid = i < n;
            int d = valid ? digit_of(keys[i], shift, mask) : 0;
            warp_count(table, d, valid);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kRadix; i += kSortThreads)
        if (table[i]) atomicAdd(&hdr->hist[0][i], (uint32_t)table[i]);
}

// Exclusive scan of 512 ints held two per thread (entries 2t, 2t+1); all 256 threads call it.
__device__ __forceinline__ void scan512(int a, int b, int* scan_tmp, int& excl_a, int& excl_b) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int s = a + b;
    int inc = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
    __syncthreads();                       // scan_tmp may still be read from a previous call
    if (lane == 31) scan_tmp[w] = inc;
    __syncthreads();
    int woff = 0;
    for (int k = 0; k < w; ++k) woff += scan_tmp[k];
    excl_a = woff + inc - s;
    excl_b = excl_a + a;
}

struct SortSmem {
    int cnt[kSortWarps][kRadix];      // per-warp digit counts, later exclusive offsets across warps
    int base[kRadix];                 // global position of the tile's first key of each digit
    int next_tab[kRadix];             // next pass's digit counts of this tile
    int tile_excl[kRadix];            // position of each digit's first key inside the sorted tile
    uint64_t skey[kSortTile];         // the tile, sorted by digit
    int32_t sval[kSortTile];
    int scan_tmp[kSortWarps];
    uint32_t tile;
};

__global__ void __launch_bounds__(kSortThreads, 2) sort_onesweep_kernel(
    const uint64_t* __restrict__ keys_in, const int32_t* __restrict__ vals_in,
    uint64_t* __restrict__ keys_out, int32_t* __restrict__ vals_out,
    const int64_t* __restrict__ n_ptr, int64_t capacity, int pass, int shift, int mask, int next_shift, int next_mask,
    SortHeader* __restrict__ hdr, uint32_t* __restrict__ desc, uint32_t* __restrict__ desc_next) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SortSmem& sm = *reinterpret_cast<SortSmem*>(smem_raw);

#ifdef SSB_SORT_PROFILE
    long long tk[7];
#define SSB_TICK(i) tk[i] = clock64()
#else
#define SSB_TICK(i)
#endif
    SSB_TICK(0);
    const int64_t n = min(*n_ptr, capacity);
    const int64_t n_tiles = (n + kSortTile - 1) / kSortTile;
    if (threadIdx.x == 0) sm.tile = atomicAdd(&hdr->ticket[pass], 1u);
    for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&sm.cnt[0][0])[i] = 0;
    for (int i = threadIdx.x; i < kRadix; i += kSortThreads) sm.next_tab[i] = 0;
    __syncthreads();
    const int64_t tile = sm.tile;
    if (tile >= n_tiles) return;
    SSB_TICK(1);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t tile_begin = tile * kSortTile;
    const int tile_count = (int)min((int64_t)kSortTile, n - tile_begin);
    const int64_t wbase = tile_begin + (int64_t)w * kSortWarpSpan;
    const int nbits = __popc((unsigned)mask);

    uint64_t key[kSortItems];
    int32_t val[kSortItems];
    int rank[kSortItems];
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        int64_t i = wbase + r * 32 + lane;
        key[r] = i < n ? keys_in[i] : 0;
    }
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        int64_t i = wbase + r * 32 + lane;
        val[r] = i < n ? vals_in[i] : 0;
    }
    // exclusive scan of the pass's digit totals -> base[] (the global loads overlap the key loads)
    {
        const int a = (int)hdr->hist[pass][2 * threadIdx.x], b = (int)hdr->hist[pass][2 * threadIdx.x + 1];
        int ea, eb;
        scan512(a, b, sm.scan_tmp, ea, eb);
        sm.base[2 * threadIdx.x] = ea;
        sm.base[2 * threadIdx.x + 1] = eb;
    }
    SSB_TICK(2);
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const bool valid = wbase + r * 32 + lane < n;
        rank[r] = warp_rank(sm.cnt[w], digit_of(key[r], shift, mask), valid, lane, nbits);
        if (next_mask != 0) warp_count(sm.next_tab, digit_of(key[r], next_shift, next_mask), valid);
    }
    SSB_TICK(3);
    __syncthreads();

    // per digit: offsets of the warps inside the tile; publish the tile's counts at once
    int tot[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int d = 2 * threadIdx.x + h;
        int run = 0;
#pragma unroll
        for (int k = 0; k < kSortWarps; ++k) { int t = sm.cnt[k][d]; sm.cnt[k][d] = run; run += t; }
        tot[h] = run;
        ((volatile uint32_t*)desc)[tile * kRadix + d] = (tile == 0 ? kFlagInclusive : kFlagAggregate) | (uint32_t)run;
    }
    {
        int ea, eb;
        scan512(tot[0], tot[1], sm.scan_tmp, ea, eb);
        sm.tile_excl[2 * threadIdx.x] = ea;
        sm.tile_excl[2 * threadIdx.x + 1] = eb;
    }
    __syncthreads();
    // stage the tile in digit order (stable: warps in order, rounds in order, lanes in order)
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        if (wbase + r * 32 + lane < n) {
            const int d = digit_of(key[r], shift, mask);
            const int lpos = sm.tile_excl[d] + sm.cnt[w][d] + rank[r];
            sm.skey[lpos] = key[r];
            sm.sval[lpos] = val[r];
        }
    }
    SSB_TICK(4);

    // look back over the predecessors, kLookWindow rows at a time: the loads of a window are
    // independent, so a run of count-only rows costs one memory latency per window, not per row
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int d = 2 * threadIdx.x + h;
        uint32_t prefix = 0;
        if (tile != 0) {
            bool done = false;
            for (int64_t t = tile - 1; t >= 0 && !done; t -= kLookWindow) {
                uint32_t v[kLookWindow];
#pragma unroll
                for (int j = 0; j < kLookWindow; ++j) {
                    const int64_t tj = t - j;
                    v[j] = tj >= 0 ? ((volatile uint32_t*)desc)[tj * kRadix + d] : (2u << 30);
                }
#pragma unroll
                for (int j = 0; j < kLookWindow; ++j) {
                    if (done) break;
                    uint32_t x = v[j];
                    if ((x >> 30) == 0u) {
                        volatile uint32_t* cell = desc + (t - j) * kRadix + d;
                        int spins = 0;
                        while (((x = *cell) >> 30) == 0u) {
                            if (++spins > kSpinLimit) { atomicExch(&hdr->error, 1u); break; }
                            __nanosleep(20);
                        }
                    }
                    prefix += x & kValueMask;
                    if ((x >> 30) != 1u) done = true;      // inclusive prefix (or gave up): stop
                }
            }
            ((volatile uint32_t*)desc)[tile * kRadix + d] = kFlagInclusive | ((prefix + (uint32_t)tot[h]) & kValueMask);
        }
        sm.base[d] += (int)prefix;
        // ready the other descriptor region for the next pass, and hand on the next digit's totals
        desc_next[tile * kRadix + d] = 0u;
        if (next_mask != 0 && sm.next_tab[d]) atomicAdd(&hdr->hist[pass + 1][d], (uint32_t)sm.next_tab[d]);
    }
    __syncthreads();
    SSB_TICK(5);

    // write out in sorted-tile order: neighbouring threads write neighbouring addresses
    for (int i = threadIdx.x; i < tile_count; i += kSortThreads) {
        const uint64_t k = sm.skey[i];
        const int d = digit_of(k, shift, mask);
        const int64_t pos = (int64_t)sm.base[d] + (i - sm.tile_excl[d]);
        keys_out[pos] = k;
        vals_out[pos] = sm.sval[i];
    }
    SSB_TICK(6);
#ifdef SSB_SORT_PROFILE
    if (threadIdx.x == 0) {
        for (int i = 0; i < 6; ++i) atomicAdd(&hdr->prof[i], (unsigned long long)(tk[i + 1] - tk[i]));
        atomicAdd(&hdr->prof[6], 1ull);
    }
#endif
}

static int64_t desc_region_words(int64_t capacity) { return ceil_div(capacity > 0 ? capacity : 1, kSortTile) * kRadix; }

// Device address of the built-in scratch array on the current device (defined with ssb_sort_pairs_u64_noalloc).
static int static_sort_scratch(void** out);

}  // namespace ssb

extern "C" {

int64_t ssb_sort_workspace_bytes(int64_t capacity) {
    using namespace ssb;
    return align_up((int64_t)sizeof(SortHeader), 256) + 2 * align_up(desc_region_words(capacity) * 4, 256);
}

int ssb_sort_pairs_u64(int64_t* d_keys_a, int32_t* d_vals_a, int64_t* d_keys_b, int32_t* d_vals_b,
                       const int64_t* d_n, int64_t capacity, int32_t begin_bit, int32_t end_bit,
                       void* d_workspace, int64_t workspace_bytes, int32_t* selector, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_keys_a && d_vals_a && d_keys_b && d_vals_b && d_n && d_workspace && selector, "ssb_sort_pairs_u64: NULL argument");
    SSB_REQUIRE(begin_bit >= 0 && end_bit <= 64 && begin_bit <= end_bit, "ssb_sort_pairs_u64: bad bit range [%d, %d)", begin_bit, end_bit);
    SSB_REQUIRE(capacity >= 0 && capacity < ((int64_t)1 << 30), "ssb_sort_pairs_u64: capacity must be below 2^30 pairs");
    SSB_REQUIRE(workspace_bytes >= ssb_sort_workspace_bytes(capacity), "ssb_sort_pairs_u64: workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    *selector = 0;
    const int total_bits = end_bit - begin_bit;
    if (total_bits == 0 || capacity == 0) return SSB_OK;
    const int passes = (total_bits + kRadixBits - 1) / kRadixBits;
    SSB_REQUIRE(passes <= kMaxPasses, "ssb_sort_pairs_u64: bit range too wide");
    int bits[kMaxPasses], shifts[kMaxPasses];
    for (int p = 0, at = begin_bit; p < passes; ++p) {
        bits[p] = total_bits / passes + (p < total_bits % passes ? 1 : 0);
        shifts[p] = at;
        at += bits[p];
    }
    char* ws = (char*)d_workspace;
    SortHeader* hdr = (SortHeader*)ws;
    const int64_t region_bytes = align_up(desc_region_words(capacity) * 4, 256);
    uint32_t* desc[2] = {(uint32_t*)(ws + align_up((int64_t)sizeof(SortHeader), 256)),
                         (uint32_t*)(ws + align_up((int64_t)sizeof(SortHeader), 256) + region_bytes)};
    if (int e = ensure_dynamic_smem((const void*)sort_onesweep_kernel, (int)sizeof(SortSmem))) return e;
    SSB_CUDA(cudaMemsetAsync(hdr, 0, sizeof(SortHeader), st));
    const int64_t tiles_cap = ceil_div(capacity, kSortTile);
    int hist_blocks = (int)(tiles_cap < 148 * 8 ? tiles_cap : 148 * 8);
    sort_first_hist_kernel<<<hist_blocks, kSortThreads, 0, st>>>((const uint64_t*)d_keys_a, d_n, capacity, shifts[0], (1 << bits[0]) - 1, hdr, desc[0]);
    SSB_LAUNCHED("sort_first_hist_kernel");
    int sel = 0;
    uint64_t* kbuf[2] = {(uint64_t*)d_keys_a, (uint64_t*)d_keys_b};
    int32_t* vbuf[2] = {d_vals_a, d_vals_b};
    for (int p = 0; p < passes; ++p) {
        const bool last = p + 1 == passes;
        sort_onesweep_kernel<<<(unsigned)tiles_cap, kSortThreads, sizeof(SortSmem), st>>>(
            kbuf[sel], vbuf[sel], kbuf[sel ^ 1], vbuf[sel ^ 1], d_n, capacity, p, shifts[p], (1 << bits[p]) - 1,
            last ? 0 : shifts[p + 1], last ? 0 : (1 << bits[p + 1]) - 1, hdr, desc[p & 1], desc[(p + 1) & 1]);
        SSB_LAUNCHED("sort_onesweep_kernel");
        sel ^= 1;
    }
    *selector = sel;
    return SSB_OK;
}

/* Non-zero if a pass of the last sort on this workspace gave up waiting on a
 * descriptor (its output is then not sorted).  Synchronises the stream. */
int ssb_sort_check(const void* d_workspace, void* stream) {
    using namespace ssb;
    if (!d_workspace) {       // the built-in scratch of ssb_sort_pairs_u64_noalloc on the current device
        void* p = nullptr;
        if (int e = static_sort_scratch(&p)) return e;
        d_workspace = p;
    }
    uint32_t err = 0;
    const SortHeader* hdr = (const SortHeader*)d_workspace;
    SSB_CUDA(cudaMemcpyAsync(&err, &hdr->error, sizeof(err), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SSB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (err) { set_error("ssb_sort_pairs_u64: a tile gave up waiting for its predecessor; the output is not sorted"); return SSB_ERR_CUDA; }
    return SSB_OK;
}


}  // extern "C"

// ---------------------------------------------------------------------------
// Sorting without a caller-provided workspace and without any allocation.
//
// Who needs it: code that is not allowed to create device memory at the point
// where it sorts -- a host application that hands a plug-in a fixed set of
// buffers and forbids it to call cudaMalloc, or a frame/step loop in which an
// allocation (which synchronises the whole device) would stall every other
// stream.  For them the sort's scratch lives in the library image itself.
// ---------------------------------------------------------------------------
namespace ssb {

constexpr int64_t kStaticSortMaxPairs = (int64_t)1 << 20;            // 1,048,576 pairs
constexpr int64_t kStaticSortTiles = kStaticSortMaxPairs / kSortTile; // 256
constexpr int64_t kStaticSortBytes = ((int64_t)sizeof(SortHeader) + 255) / 256 * 256 + 2 * kStaticSortTiles * kRadix * 4;

// Held by every GPU that loads the library, from load until the process exits (about 1 MB).
static __device__ __align__(256) unsigned char g_static_sort_scratch[kStaticSortBytes];

}  // namespace ssb

#include <mutex>

namespace ssb {

// The array's name is only a host-side handle; the kernels need its address in the
// current device's memory, looked up once per device and remembered.
static int static_sort_scratch(void** out) {
    static std::mutex mu;
    static void* scratch_of_device[kMaxDevices] = {nullptr};
    int dev = -1;
    SSB_CUDA(cudaGetDevice(&dev));
    SSB_REQUIRE(dev >= 0 && dev < kMaxDevices, "ssb_sort_pairs_u64_noalloc: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!scratch_of_device[dev]) {
        void* p = nullptr;
        SSB_CUDA(cudaGetSymbolAddress(&p, g_static_sort_scratch));
        scratch_of_device[dev] = p;
    }
    *out = scratch_of_device[dev];
    return SSB_OK;
}

}  // namespace ssb

extern "C" int ssb_sort_pairs_u64_noalloc(int64_t* d_keys_a, int32_t* d_vals_a, int64_t* d_keys_b, int32_t* d_vals_b,
                                          const int64_t* d_n, int64_t capacity, int32_t begin_bit, int32_t end_bit,
                                          int32_t* selector, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(capacity >= 0, "ssb_sort_pairs_u64_noalloc: negative capacity %lld", (long long)capacity);
    if (capacity > kStaticSortMaxPairs) {
        set_error("ssb_sort_pairs_u64_noalloc: capacity %lld exceeds the built-in scratch, which serves at most %lld pairs; "
                  "use ssb_sort_pairs_u64 with a workspace of your own", (long long)capacity, (long long)kStaticSortMaxPairs);
        return SSB_ERR_CAPACITY;
    }
    void* scratch = nullptr;
    if (int e = static_sort_scratch(&scratch)) return e;
    return ssb_sort_pairs_u64(d_keys_a, d_vals_a, d_keys_b, d_vals_b, d_n, capacity, begin_bit, end_bit,
                              scratch, kStaticSortBytes, selector, stream);
}
