// splat.ply: the inference artefact spirula-studio writes next to every checkpoint, and reading one back.
//
// The file is the property layout of the original 3D Gaussian Splatting release (x y z / nx ny nz / f_dc_0..2 /
// f_rest_0..44 / opacity / scale_0..2 / rot_0..3, binary little endian, 62 floats per vertex), values raw: log scales,
// logit opacity, (w, x, y, z) rotation, DC as the SH coefficient.  The reference builds it on the host from full copies
// of every array (src/engine/EngineCheckpoint.cpp:130-330): it drops splats with a non-finite parameter and splats whose
// opacity logit is below logit(1/255) = -5.5373, dequantises the SH values, and stores the SH rest channel-major
// (r0..r14, g0..g14, b0..b14) where the engine keeps it coefficient-major.
//
// Here the rows are made on the device: one pass marks what is kept and counts per block of 256 splats, one scan turns
// the counts into row numbers (kept splats stay in their order), and a row kernel writes finished 248-byte rows for a
// range of splats into a buffer that goes to the file through two pinned staging buffers -- while one range is on its
// way to the host the next is being assembled and the previous one written.  The host never sees a filtered-out splat and
// needs a fixed 65 MB of pinned memory whatever the scene's size.
//
// The reader follows the reference's (src/checkpoint/SplatPly.cpp:65-254): any order and any scalar type of the vertex
// properties, binary little endian or ASCII, other elements ignored, a list property on the vertex element refused; it
// needs x y z, opacity, scale_*, rot_*, f_dc_*; f_rest_* give the SH degree (0 when absent) and are transposed back.
#include "ssb_common.cuh"

#include <algorithm>
#include <cctype>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace ssb {

constexpr int kPlyBlock = 256;
constexpr int kPlyRowFloats = 3 + 3 + 3 + 3 * kNumSh + 1 + 3 + 4;     // 62
constexpr int64_t kPlyRange = 131072;                                 // splats per staged range (32.5 MB of rows at most)
constexpr float kPlyOpacityMin = -5.5373f;                            // logit(1/255), as the reference writes it

__device__ __forceinline__ float ply_sh_value(const SsbSplats& p, const SsbShQuant& q, int64_t splat, int j, int ch) {
    const int64_t cell = splat * (3 * kNumSh) + 3 * j + ch;
    if (q.packed == nullptr) return p.features_sh[cell];
    const int64_t b = cell / q.bounds_stride;
    const float lo = q.bounds[2 * b], hi = q.bounds[2 * b + 1];
    if (q.bits == 8) return lo + (hi - lo) * ((float)((const uint8_t*)q.packed)[cell] * (1.0f / 255.0f));
    return lo + (hi - lo) * ((float)((const uint16_t*)q.packed)[cell] * (1.0f / 65535.0f));
}

// keep[i] = every parameter finite (quantised SH values are finite by construction and are not looked at) and the
// opacity logit not below the threshold; counts[block] = kept splats of the block
__global__ void __launch_bounds__(kPlyBlock) ply_keep_kernel(SsbSplats p, int fp32_sh, int64_t n, uint8_t* __restrict__ keep,
                                                             int32_t* __restrict__ counts) {
    const int64_t i = (int64_t)blockIdx.x * kPlyBlock + threadIdx.x;
    bool ok = false;
    if (i < n) {
        ok = true;
#pragma unroll
        for (int k = 0; k < 3; ++k) ok = ok && isfinite(p.means[3 * i + k]) && isfinite(p.scales[3 * i + k]) && isfinite(p.features_dc[3 * i + k]);
#pragma unroll
        for (int k = 0; k < 4; ++k) ok = ok && isfinite(p.quats[4 * i + k]);
        const float o = p.opacities[i];
        ok = ok && isfinite(o);
        if (ok && fp32_sh)
            for (int k = 0; k < 3 * kNumSh; ++k) ok = ok && isfinite(p.features_sh[i * (3 * kNumSh) + k]);
        ok = ok && !(o < kPlyOpacityMin);
        keep[i] = ok ? 1 : 0;
    }
    const int c = __syncthreads_count(ok);
    if (threadIdx.x == 0) counts[blockIdx.x] = c;
}

// offsets[b] = kept splats before block b (int64), offsets[n_blocks] = all of them; one CTA walks the blocks
__global__ void __launch_bounds__(1024) ply_scan_kernel(const int32_t* __restrict__ counts, int64_t n_blocks, int64_t* __restrict__ offsets) {
    __shared__ int64_t warp_tot[32];
    __shared__ int64_t carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int64_t base = 0; base < n_blocks; base += 1024) {
        const int64_t b = base + threadIdx.x;
        const int64_t v = b < n_blocks ? counts[b] : 0;
        int64_t incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int64_t t = __shfl_up_sync(0xffffffffu, incl, o); if ((threadIdx.x & 31) >= o) incl += t; }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = incl;
        __syncthreads();
        int64_t before = carry_s;
        for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) before += warp_tot[w];
        if (b < n_blocks) offsets[b] = before + incl - v;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = before + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) offsets[n_blocks] = carry_s;
}

// rows of the kept splats of blocks [first_block, ...) of one range, numbered from the range's first kept splat
__global__ void __launch_bounds__(kPlyBlock) ply_rows_kernel(SsbSplats p, SsbShQuant q, int64_t n, const uint8_t* __restrict__ keep,
                                                             const int64_t* __restrict__ offsets, int64_t first_block, float* __restrict__ rows) {
    __shared__ int warp_cnt[kPlyBlock / 32];
    const int64_t block = first_block + blockIdx.x;
    const int64_t i = block * kPlyBlock + threadIdx.x;
    const bool k = i < n && keep[i] != 0;
    const unsigned bal = __ballot_sync(0xffffffffu, k);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) warp_cnt[w] = __popc(bal);
    __syncthreads();
    if (!k) return;
    int rank = __popc(bal & ((1u << lane) - 1u));
    for (int v = 0; v < w; ++v) rank += warp_cnt[v];
    float* row = rows + (offsets[block] - offsets[first_block] + rank) * kPlyRowFloats;
    int c = 0;
    row[c++] = p.means[3 * i]; row[c++] = p.means[3 * i + 1]; row[c++] = p.means[3 * i + 2];
    row[c++] = 0.f; row[c++] = 0.f; row[c++] = 0.f;                                   // nx ny nz
    row[c++] = p.features_dc[3 * i]; row[c++] = p.features_dc[3 * i + 1]; row[c++] = p.features_dc[3 * i + 2];
    for (int ch = 0; ch < 3; ++ch)                                                    // channel-major in the file
        for (int j = 0; j < kNumSh; ++j) row[c++] = ply_sh_value(p, q, i, j, ch);
    row[c++] = p.opacities[i];
    row[c++] = p.scales[3 * i]; row[c++] = p.scales[3 * i + 1]; row[c++] = p.scales[3 * i + 2];
    row[c++] = p.quats[4 * i]; row[c++] = p.quats[4 * i + 1]; row[c++] = p.quats[4 * i + 2]; row[c++] = p.quats[4 * i + 3];
}

namespace {

enum PlyType { F32, F64, I8, U8, I16, U16, I32, U32 };
struct PlyProp { std::string name; PlyType type; size_t offset; };
struct PlyHeader {
    bool ok = false, binary_le = false, ascii = false;
    int64_t num_vertex = 0;
    std::vector<PlyProp> props;
    size_t row_bytes = 0;
    long data_start = 0;
};

size_t ply_type_size(PlyType t) { return t == F64 ? 8 : (t == I8 || t == U8) ? 1 : (t == I16 || t == U16) ? 2 : 4; }

bool ply_parse_type(const std::string& s, PlyType& out) {
    static const struct { const char* a; const char* b; PlyType t; } names[] = {
        {"float", "float32", F32}, {"double", "float64", F64}, {"char", "int8", I8}, {"uchar", "uint8", U8},
        {"short", "int16", I16}, {"ushort", "uint16", U16}, {"int", "int32", I32}, {"uint", "uint32", U32}};
    for (const auto& e : names) if (s == e.a || s == e.b) { out = e.t; return true; }
    return false;
}

bool read_line(FILE* f, std::string& line) {
    line.clear();
    int ch;
    bool any = false;
    while ((ch = std::fgetc(f)) != EOF) {
        any = true;
        if (ch == '\n') break;
        if (line.size() >= 4096) return false;      // no header line is this long: not a PLY (do not swallow a binary file)
        line.push_back((char)ch);
    }
    if (!line.empty() && line.back() == '\r') line.pop_back();
    return any;
}

std::vector<std::string> split_ws(const std::string& s) {
    std::vector<std::string> out;
    size_t i = 0;
    while (i < s.size()) {
        while (i < s.size() && std::isspace((unsigned char)s[i])) ++i;
        size_t j = i;
        while (j < s.size() && !std::isspace((unsigned char)s[j])) ++j;
        if (j > i) out.push_back(s.substr(i, j - i));
        i = j;
    }
    return out;
}

// A malformed file comes back with ok == false (src/checkpoint/SplatPly.cpp:65-112)
PlyHeader ply_read_header(FILE* f) {
    PlyHeader h;
    std::string line;
    if (!read_line(f, line) || line.rfind("ply", 0) != 0) return h;
    bool in_vertex = false;
    while (read_line(f, line)) {
        const std::vector<std::string> t = split_ws(line);
        if (t.empty()) continue;
        if (t[0] == "format") {
            h.binary_le = t.size() > 1 && t[1] == "binary_little_endian";
            h.ascii = t.size() > 1 && t[1] == "ascii";
        } else if (t[0] == "element") {
            in_vertex = t.size() > 1 && t[1] == "vertex";
            if (in_vertex) h.num_vertex = t.size() > 2 ? std::atoll(t[2].c_str()) : 0;
        } else if (t[0] == "property") {
            if (t.size() > 1 && t[1] == "list") {      // no fixed width: a vertex element with one cannot be strided
                if (in_vertex) return h;
                continue;
            }
            if (!in_vertex) continue;
            PlyProp p;
            if (t.size() < 3 || !ply_parse_type(t[1], p.type)) return h;
            p.name = t[2];
            p.offset = h.row_bytes;
            h.row_bytes += ply_type_size(p.type);
            h.props.push_back(p);
        } else if (t[0] == "end_header") {
            h.data_start = std::ftell(f);
            h.ok = h.num_vertex >= 0 && !h.props.empty() && (h.binary_le || h.ascii);
            return h;
        }
    }
    return h;
}

int ply_find(const PlyHeader& h, const std::string& name) {
    for (size_t i = 0; i < h.props.size(); ++i) if (h.props[i].name == name) return (int)i;
    return -1;
}

float ply_scalar(const uint8_t* row, const PlyProp& p) {
    const uint8_t* q = row + p.offset;
    switch (p.type) {
        case F32: { float v; std::memcpy(&v, q, 4); return v; }
        case F64: { double v; std::memcpy(&v, q, 8); return (float)v; }
        case I8: { int8_t v; std::memcpy(&v, q, 1); return (float)v; }
        case U8: { uint8_t v; std::memcpy(&v, q, 1); return (float)v; }
        case I16: { int16_t v; std::memcpy(&v, q, 2); return (float)v; }
        case U16: { uint16_t v; std::memcpy(&v, q, 2); return (float)v; }
        case I32: { int32_t v; std::memcpy(&v, q, 4); return (float)v; }
        case U32: { uint32_t v; std::memcpy(&v, q, 4); return (float)v; }
    }
    return 0.0f;
}

const char* const kSplatProps[] = {"x", "y", "z", "opacity", "scale_0", "scale_1", "scale_2", "rot_0", "rot_1", "rot_2", "rot_3",
                                   "f_dc_0", "f_dc_1", "f_dc_2"};

// number of f_rest_<i> columns counted from 0 without a gap, and the SH degree they make (-1: not a whole degree)
int ply_rest_degree(const PlyHeader& h, std::vector<int>* cols) {
    int n_rest = 0;
    for (;; ++n_rest) {
        const int c = ply_find(h, "f_rest_" + std::to_string(n_rest));
        if (c < 0) break;
        if (cols) cols->push_back(c);
    }
    if (n_rest == 0) return 0;
    if (n_rest % 3 != 0) return -1;
    for (int deg = 1; deg <= 4; ++deg) if (n_rest / 3 == (deg + 1) * (deg + 1) - 1) return deg;
    return -1;
}

}  // namespace
}  // namespace ssb

extern "C" {

int ssb_ply_write(const char* path, const SsbSplats* params, const SsbShQuant* shq, int64_t n, int64_t* kept_out, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(path && params && n >= 0, "ssb_ply_write: bad argument");
    SSB_REQUIRE(params->means && params->quats && params->scales && params->opacities && params->features_dc, "ssb_ply_write: parameter arrays missing");
    SsbShQuant q = {nullptr, nullptr, 32, 0, 256};
    if (shq && shq->packed && (shq->bits == 8 || shq->bits == 16)) {
        q = *shq;
        SSB_REQUIRE(q.bounds != nullptr, "ssb_ply_write: quantised SH needs its bounds");
        if (q.bounds_stride <= 0) q.bounds_stride = (int64_t)256 * 3 * kNumSh;
    } else {
        SSB_REQUIRE(params->features_sh != nullptr, "ssb_ply_write: features_sh is NULL and no quantised SH was given");
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t n_blocks = ceil_div(n, kPlyBlock);
    uint8_t* d_keep = nullptr;
    int32_t* d_counts = nullptr;
    int64_t* d_offsets = nullptr;
    float* d_rows[2] = {nullptr, nullptr};
    char* h_stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    FILE* f = nullptr;
    std::vector<int64_t> offsets((size_t)n_blocks + 1, 0);
    int rc = SSB_OK;
    const size_t range_bytes = (size_t)kPlyRange * kPlyRowFloats * sizeof(float);
    auto cleanup = [&]() {
        cudaFree(d_keep); cudaFree(d_counts); cudaFree(d_offsets);
        for (int k = 0; k < 2; ++k) {
            cudaFree(d_rows[k]);
            if (h_stage[k]) cudaFreeHost(h_stage[k]);
            if (done[k]) cudaEventDestroy(done[k]);
        }
        if (f) std::fclose(f);
    };
#define SSB_PLY_TRY(call, code, what) do { if ((call) != cudaSuccess) { cudaGetLastError(); set_error("ssb_ply_write: %s failed", what); rc = code; cleanup(); return rc; } } while (0)
    if (n > 0) {
        SSB_PLY_TRY(cudaMalloc(&d_keep, (size_t)n), SSB_ERR_OUT_OF_MEMORY, "cudaMalloc");
        SSB_PLY_TRY(cudaMalloc(&d_counts, (size_t)n_blocks * 4), SSB_ERR_OUT_OF_MEMORY, "cudaMalloc");
        SSB_PLY_TRY(cudaMalloc(&d_offsets, ((size_t)n_blocks + 1) * 8), SSB_ERR_OUT_OF_MEMORY, "cudaMalloc");
        ply_keep_kernel<<<(unsigned)n_blocks, kPlyBlock, 0, st>>>(*params, q.packed == nullptr ? 1 : 0, n, d_keep, d_counts);
        ply_scan_kernel<<<1, 1024, 0, st>>>(d_counts, n_blocks, d_offsets);
        SSB_PLY_TRY(cudaMemcpyAsync(offsets.data(), d_offsets, ((size_t)n_blocks + 1) * 8, cudaMemcpyDeviceToHost, st), SSB_ERR_CUDA, "cudaMemcpyAsync");
        SSB_PLY_TRY(cudaStreamSynchronize(st), SSB_ERR_CUDA, "the keep pass");
    }
    const int64_t kept = offsets[(size_t)n_blocks];
    if (kept_out) *kept_out = kept;
    f = std::fopen(path, "wb");
    if (!f) { set_error("ssb_ply_write: cannot open '%s' for writing", path); cleanup(); return SSB_ERR_IO; }
    // the header, line for line as the reference writes it (src/engine/EngineCheckpoint.cpp:300-310)
    std::string hdr = "ply\nformat binary_little_endian 1.0\nelement vertex " + std::to_string(kept) + "\n";
    hdr += "property float x\nproperty float y\nproperty float z\nproperty float nx\nproperty float ny\nproperty float nz\n";
    hdr += "property float f_dc_0\nproperty float f_dc_1\nproperty float f_dc_2\n";
    for (int j = 0; j < 3 * kNumSh; ++j) hdr += "property float f_rest_" + std::to_string(j) + "\n";
    hdr += "property float opacity\nproperty float scale_0\nproperty float scale_1\nproperty float scale_2\n";
    hdr += "property float rot_0\nproperty float rot_1\nproperty float rot_2\nproperty float rot_3\nend_header\n";
    bool io_ok = std::fwrite(hdr.data(), 1, hdr.size(), f) == hdr.size();
    if (kept > 0) {
        for (int k = 0; k < 2; ++k) {
            SSB_PLY_TRY(cudaMalloc(&d_rows[k], range_bytes), SSB_ERR_OUT_OF_MEMORY, "cudaMalloc");
            SSB_PLY_TRY(cudaMallocHost((void**)&h_stage[k], range_bytes), SSB_ERR_OUT_OF_MEMORY, "cudaMallocHost");
            SSB_PLY_TRY(cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming), SSB_ERR_CUDA, "cudaEventCreate");
        }
        const int64_t blocks_per_range = kPlyRange / kPlyBlock;
        const int64_t n_ranges = ceil_div(n_blocks, blocks_per_range);
        auto range_rows = [&](int64_t r) {
            const int64_t b0 = r * blocks_per_range, b1 = std::min(n_blocks, b0 + blocks_per_range);
            return offsets[(size_t)b1] - offsets[(size_t)b0];
        };
        auto start = [&](int64_t r) {       // assemble range r and send it towards staging buffer r & 1
            const int64_t b0 = r * blocks_per_range, b1 = std::min(n_blocks, b0 + blocks_per_range);
            const int64_t rows = range_rows(r);
            if (rows > 0) {
                ply_rows_kernel<<<(unsigned)(b1 - b0), kPlyBlock, 0, st>>>(*params, q, n, d_keep, d_offsets, b0, d_rows[r & 1]);
                if (cudaMemcpyAsync(h_stage[r & 1], d_rows[r & 1], (size_t)rows * kPlyRowFloats * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess) return false;
            }
            return cudaEventRecord(done[r & 1], st) == cudaSuccess;
        };
        bool ok = start(0);
        for (int64_t r = 0; ok && r < n_ranges; ++r) {
            if (r + 1 < n_ranges) ok = start(r + 1);
            if (ok) ok = cudaEventSynchronize(done[r & 1]) == cudaSuccess;
            const size_t bytes = (size_t)range_rows(r) * kPlyRowFloats * sizeof(float);
            if (ok && bytes && io_ok) io_ok = std::fwrite(h_stage[r & 1], 1, bytes, f) == bytes;
        }
        if (!ok) {
            cudaStreamSynchronize(st);
            cudaGetLastError();
            set_error("ssb_ply_write: a device step failed");
            cleanup();
            return SSB_ERR_CUDA;
        }
    }
#undef SSB_PLY_TRY
    if (std::fflush(f) != 0) io_ok = false;
    cleanup();
    if (!io_ok) { set_error("ssb_ply_write: writing '%s' failed", path); return SSB_ERR_IO; }
    return SSB_OK;
}

int ssb_ply_info(const char* path, int64_t* num, int32_t* sh_degree) {
    using namespace ssb;
    SSB_REQUIRE(path, "ssb_ply_info: NULL path");
    FILE* f = std::fopen(path, "rb");
    if (!f) { set_error("ssb_ply_info: cannot open '%s'", path); return SSB_ERR_IO; }
    const PlyHeader h = ply_read_header(f);
    std::fclose(f);
    bool splat = h.ok;
    for (const char* name : kSplatProps) splat = splat && ply_find(h, name) >= 0;
    if (!splat) { set_error("ssb_ply_info: '%s' is not a 3D Gaussian Splatting PLY", path); return SSB_ERR_UNSUPPORTED; }
    const int deg = ply_rest_degree(h, nullptr);
    if (deg < 0) { set_error("ssb_ply_info: '%s': the f_rest properties do not make a whole SH degree", path); return SSB_ERR_UNSUPPORTED; }
    if (num) *num = h.num_vertex;
    if (sh_degree) *sh_degree = deg;
    return SSB_OK;
}

int ssb_ply_read(const char* path, int64_t num, int32_t sh_degree, float* means, float* quats, float* scales, float* opacities,
                 float* features_dc, float* features_sh) {
    using namespace ssb;
    SSB_REQUIRE(path && means && quats && scales && opacities && features_dc, "ssb_ply_read: NULL argument");
    FILE* f = std::fopen(path, "rb");
    if (!f) { set_error("ssb_ply_read: cannot open '%s'", path); return SSB_ERR_IO; }
    const PlyHeader h = ply_read_header(f);
    auto bail = [&](int code, const char* what) { std::fclose(f); set_error("ssb_ply_read: '%s': %s", path, what); return code; };
    if (!h.ok) return bail(SSB_ERR_UNSUPPORTED, "not a readable PLY");
    int col[14];
    for (int k = 0; k < 14; ++k) {
        col[k] = ply_find(h, kSplatProps[k]);
        if (col[k] < 0) return bail(SSB_ERR_UNSUPPORTED, "a 3D Gaussian Splatting property is missing");
    }
    std::vector<int> crest;
    const int deg = ply_rest_degree(h, &crest);
    if (deg < 0) return bail(SSB_ERR_UNSUPPORTED, "the f_rest properties do not make a whole SH degree");
    if (num != h.num_vertex || sh_degree != deg) return bail(SSB_ERR_INVALID_ARGUMENT, "vertex count or SH degree differ from the caller's (ssb_ply_info)");
    const int64_t K = features_sh ? (int64_t)(deg + 1) * (deg + 1) - 1 : 0;       // features_sh NULL: the f_rest columns are skipped
    const int64_t n = h.num_vertex;
    const size_t n_props = h.props.size();
    std::vector<float> vals(n_props);
    auto take = [&](int64_t i) {
        means[3 * i] = vals[col[0]]; means[3 * i + 1] = vals[col[1]]; means[3 * i + 2] = vals[col[2]];
        opacities[i] = vals[col[3]];
        for (int k = 0; k < 3; ++k) scales[3 * i + k] = vals[col[4 + k]];
        for (int k = 0; k < 4; ++k) quats[4 * i + k] = vals[col[7 + k]];
        for (int k = 0; k < 3; ++k) features_dc[3 * i + k] = vals[col[11 + k]];
        for (int ch = 0; ch < 3 && K > 0; ++ch)        // channel-major in the file, coefficient-major here
            for (int64_t j = 0; j < K; ++j) features_sh[(i * K + j) * 3 + ch] = vals[crest[(size_t)(ch * K + j)]];
    };
    std::fseek(f, h.data_start, SEEK_SET);
    if (h.ascii) {
        for (int64_t i = 0; i < n; ++i) {
            for (size_t k = 0; k < n_props; ++k)
                if (std::fscanf(f, "%f", &vals[k]) != 1) return bail(SSB_ERR_IO, "truncated vertex data");
            take(i);
        }
    } else {
        const int64_t kRows = 1 << 14;
        std::vector<uint8_t> raw(h.row_bytes * (size_t)kRows);
        for (int64_t row = 0; row < n; row += kRows) {
            const int64_t nr = std::min(kRows, n - row);
            if (std::fread(raw.data(), h.row_bytes, (size_t)nr, f) != (size_t)nr) return bail(SSB_ERR_IO, "truncated vertex data");
            for (int64_t i = 0; i < nr; ++i) {
                const uint8_t* r = raw.data() + (size_t)i * h.row_bytes;
                for (size_t k = 0; k < n_props; ++k) vals[k] = ply_scalar(r, h.props[k]);
                take(row + i);
            }
        }
    }
    std::fclose(f);
    return SSB_OK;
}

}  // extern "C"
