// Checkpoint container: one POSIX ustar archive ("state.tar") holding a small
// state.json followed by one flat, typed NPY v1.0 array per saved buffer.
//
// The byte layout follows spirula-studio's writer so that either side reads the
// other's files: member headers as src/core/CheckpointIO.h:53-81 writes them
// (mode 0644, uid/gid/mtime 0, octal size or GNU base-256 above 8 GiB, checksum as
// six octal digits + NUL + space, typeflag '0', magic "ustar\0" "00"), array
// headers as src/core/CheckpointIO.h:33-50 (dict with a one-dimensional shape,
// padded with spaces so that the data starts on a 64-byte boundary), members
// padded to 512 bytes and two zero blocks at the end (src/core/CheckpointIO.h:84-101).
// The reader accepts what the reference's reader accepts (src/core/CheckpointIO.h:140-212):
// octal and base-256 sizes, NPY v1 and v2/v3 header lengths.
//
// Device buffers move through two pinned staging buffers: while one chunk is on
// its way from the GPU the previous one is written to the file (and the other
// way round on load), so a save runs at the slower of the PCIe copy and the file
// system instead of their sum, and needs no device memory and a fixed amount of host memory.
#include "ssb_common.cuh"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr size_t kChunk = size_t(32) << 20;   // staging chunk, as the reference's 32 MiB host buffer

struct DTypeInfo { const char* descr; size_t size; };

// Same order as the reference's NpyScalar tags (src/core/Tensor.h:26, 45-59).
bool dtype_info(int dtype, DTypeInfo* out) {
    static const DTypeInfo table[] = {{"|u1", 1}, {"<u2", 2}, {"<u4", 4}, {"<u8", 8}, {"<i4", 4},
                                      {"<i8", 8}, {"<f2", 2}, {"<f4", 4}, {"<f8", 8}, {"|b1", 1}};
    if (dtype < 0 || dtype >= int(sizeof(table) / sizeof(table[0]))) return false;
    *out = table[dtype];
    return true;
}

std::string array_header(const char* descr, uint64_t numel) {
    std::string dict = std::string("{'descr': '") + descr + "', 'fortran_order': False, 'shape': (" +
                       std::to_string(numel) + ",), }";
    const size_t unpadded = 10 + dict.size() + 1;
    dict.append((64 - unpadded % 64) % 64, ' ');
    dict.push_back('\n');
    std::string h("\x93NUMPY\x01", 7);
    h.push_back('\0');
    h.push_back(char(dict.size() & 0xff));
    h.push_back(char((dict.size() >> 8) & 0xff));
    return h + dict;
}

void octal(char* dst, int digits, uint64_t v) {   // `digits` octal digits, most significant first, then NUL
    for (int i = digits - 1; i >= 0; --i) { dst[i] = char('0' + (v & 7)); v >>= 3; }
    dst[digits] = '\0';
}

void member_header(char h[512], const char* name, uint64_t size) {
    std::memset(h, 0, 512);
    std::strncpy(h, name, 99);
    octal(h + 100, 7, 0644);
    octal(h + 108, 7, 0);
    octal(h + 116, 7, 0);
    if (size <= 077777777777ull) {
        octal(h + 124, 11, size);
    } else {
        h[124] = char(0x80);
        for (int i = 135; i >= 125; --i) { h[i] = char(size & 0xff); size >>= 8; }
    }
    octal(h + 136, 11, 0);
    std::memset(h + 148, ' ', 8);
    h[156] = '0';
    std::memcpy(h + 257, "ustar", 5);
    h[263] = '0';
    h[264] = '0';
    unsigned sum = 0;
    for (int i = 0; i < 512; ++i) sum += (unsigned char)h[i];
    octal(h + 148, 6, sum & 0777777u);
    h[155] = ' ';
}

struct Staging {
    char* buf[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    int ensure() {
        for (int i = 0; i < 2; ++i) {
            if (!buf[i] && cudaMallocHost((void**)&buf[i], kChunk) != cudaSuccess) { cudaGetLastError(); return SSB_ERR_OUT_OF_MEMORY; }
            if (!done[i] && cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return SSB_ERR_CUDA; }
        }
        return SSB_OK;
    }
    void release() {
        for (int i = 0; i < 2; ++i) {
            if (buf[i]) cudaFreeHost(buf[i]);
            if (done[i]) cudaEventDestroy(done[i]);
            buf[i] = nullptr;
            done[i] = nullptr;
        }
    }
};

struct Member { std::string name; uint64_t offset, size; };

template <class... Args>
int fail(int code, const char* fmt, Args... args) {
    ssb::set_error(fmt, args...);
    return code;
}

}  // namespace

struct SsbCkptWriter {
    FILE* f = nullptr;
    Staging stage;
    bool failed = false;
    bool put(const void* p, size_t n) {
        if (n && std::fwrite(p, 1, n, f) != n) failed = true;
        return !failed;
    }
    bool pad(uint64_t size) {
        static const char zeros[512] = {0};
        return put(zeros, size_t((512 - size % 512) % 512));
    }
};

struct SsbCkptReader {
    FILE* f = nullptr;
    Staging stage;
    std::vector<Member> members;
    const Member* find(const char* name) const {
        for (const Member& m : members) if (m.name == name) return &m;
        return nullptr;
    }
};

namespace {

bool seek_to(FILE* f, uint64_t off) { return fseeko(f, off_t(off), SEEK_SET) == 0; }

// Where the array data of an NPY member starts, how many bytes it has, and its descr string.
int locate_array(SsbCkptReader* r, const Member& m, uint64_t* data_off, uint64_t* data_bytes, std::string* descr) {
    unsigned char pre[12];
    if (m.size < 10 || !seek_to(r->f, m.offset) || std::fread(pre, 1, 10, r->f) != 10) return SSB_ERR_IO;
    if (std::memcmp(pre, "\x93NUMPY", 6) != 0) return SSB_ERR_INVALID_ARGUMENT;
    uint64_t hlen = pre[8] | (uint64_t(pre[9]) << 8), prefix = 10;
    if (pre[6] >= 2) {
        if (std::fread(pre + 10, 1, 2, r->f) != 2) return SSB_ERR_IO;
        hlen |= (uint64_t(pre[10]) << 16) | (uint64_t(pre[11]) << 24);
        prefix = 12;
    }
    if (prefix + hlen > m.size) return SSB_ERR_INVALID_ARGUMENT;
    std::string dict(size_t(hlen), '\0');
    if (hlen && std::fread(&dict[0], 1, size_t(hlen), r->f) != hlen) return SSB_ERR_IO;
    descr->clear();
    size_t d = dict.find("'descr':");
    if (d != std::string::npos) {
        size_t q1 = dict.find('\'', d + 8);
        size_t q2 = q1 == std::string::npos ? q1 : dict.find('\'', q1 + 1);
        if (q2 != std::string::npos) *descr = dict.substr(q1 + 1, q2 - q1 - 1);
    }
    *data_off = m.offset + prefix + hlen;
    *data_bytes = m.size - prefix - hlen;
    return SSB_OK;
}

}  // namespace

extern "C" {

int ssb_ckpt_array_header(int dtype, uint64_t numel, void* out, int capacity) {
    DTypeInfo dt;
    if (!dtype_info(dtype, &dt) || !out) return SSB_ERR_INVALID_ARGUMENT;
    const std::string h = array_header(dt.descr, numel);
    if (int(h.size()) > capacity) return SSB_ERR_CAPACITY;
    std::memcpy(out, h.data(), h.size());
    return int(h.size());
}

int ssb_ckpt_member_header(const char* name, uint64_t size, void* out512) {
    if (!name || !out512 || std::strlen(name) > 99) return SSB_ERR_INVALID_ARGUMENT;
    member_header((char*)out512, name, size);
    return SSB_OK;
}

int ssb_ckpt_writer_open(const char* path, SsbCkptWriter** out) {
    if (!path || !out) return SSB_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    FILE* f = std::fopen(path, "wb");
    if (!f) return fail(SSB_ERR_IO, "checkpoint: cannot create %s", path);
    SsbCkptWriter* w = new SsbCkptWriter;
    w->f = f;
    *out = w;
    return SSB_OK;
}

int ssb_ckpt_write_bytes(SsbCkptWriter* w, const char* name, const void* data, uint64_t size) {
    if (!w || !name || (!data && size) || std::strlen(name) > 99) return SSB_ERR_INVALID_ARGUMENT;
    char h[512];
    member_header(h, name, size);
    w->put(h, 512);
    w->put(data, size_t(size));
    w->pad(size);
    return w->failed ? fail(SSB_ERR_IO, "checkpoint: write failed at member '%s'", name) : SSB_OK;
}

int ssb_ckpt_write_host(SsbCkptWriter* w, const char* name, const void* h_ptr, uint64_t nbytes, int dtype) {
    DTypeInfo dt;
    if (!w || !name || (!h_ptr && nbytes) || std::strlen(name) > 99 || !dtype_info(dtype, &dt) || nbytes % dt.size)
        return SSB_ERR_INVALID_ARGUMENT;
    const std::string hdr = array_header(dt.descr, nbytes / dt.size);
    char h[512];
    member_header(h, name, hdr.size() + nbytes);
    w->put(h, 512);
    w->put(hdr.data(), hdr.size());
    w->put(h_ptr, size_t(nbytes));
    w->pad(hdr.size() + nbytes);
    return w->failed ? fail(SSB_ERR_IO, "checkpoint: write failed at member '%s'", name) : SSB_OK;
}

int ssb_ckpt_write_device(SsbCkptWriter* w, const char* name, const void* d_ptr, uint64_t nbytes, int dtype, void* stream) {
    DTypeInfo dt;
    if (!w || !name || (!d_ptr && nbytes) || std::strlen(name) > 99 || !dtype_info(dtype, &dt) || nbytes % dt.size)
        return SSB_ERR_INVALID_ARGUMENT;
    if (int rc = w->stage.ensure()) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const std::string hdr = array_header(dt.descr, nbytes / dt.size);
    const uint64_t member = hdr.size() + nbytes;
    char h[512];
    member_header(h, name, member);
    w->put(h, 512);
    w->put(hdr.data(), hdr.size());
    // chunk k is copied into staging buffer k & 1 while chunk k - 1 goes to the file
    const char* src = (const char*)d_ptr;
    const uint64_t n_chunks = (nbytes + kChunk - 1) / kChunk;
    auto chunk_bytes = [&](uint64_t k) { return size_t(std::min<uint64_t>(kChunk, nbytes - k * kChunk)); };
    auto start = [&](uint64_t k) {
        if (cudaMemcpyAsync(w->stage.buf[k & 1], src + k * kChunk, chunk_bytes(k), cudaMemcpyDeviceToHost, st) != cudaSuccess) return false;
        return cudaEventRecord(w->stage.done[k & 1], st) == cudaSuccess;
    };
    bool ok = n_chunks == 0 || start(0);
    for (uint64_t k = 0; ok && k < n_chunks; ++k) {
        if (k + 1 < n_chunks) ok = start(k + 1);
        if (ok) ok = cudaEventSynchronize(w->stage.done[k & 1]) == cudaSuccess;
        if (ok) w->put(w->stage.buf[k & 1], chunk_bytes(k));
    }
    if (!ok) {
        cudaStreamSynchronize(st);
        cudaGetLastError();
        w->failed = true;
        return SSB_ERR_CUDA;
    }
    w->pad(member);
    return w->failed ? fail(SSB_ERR_IO, "checkpoint: write failed at member '%s'", name) : SSB_OK;
}

int ssb_ckpt_writer_close(SsbCkptWriter* w) {
    if (!w) return SSB_ERR_INVALID_ARGUMENT;
    static const char zeros[1024] = {0};
    w->put(zeros, 1024);
    if (std::fclose(w->f) != 0) w->failed = true;
    w->stage.release();
    const bool failed = w->failed;
    delete w;
    return failed ? fail(SSB_ERR_IO, "checkpoint: write failed") : SSB_OK;
}

int ssb_ckpt_reader_open(const char* path, SsbCkptReader** out) {
    if (!path || !out) return SSB_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(SSB_ERR_IO, "checkpoint: cannot open %s", path);
    SsbCkptReader* r = new SsbCkptReader;
    r->f = f;
    unsigned char h[512];
    uint64_t pos = 0;
    while (seek_to(f, pos) && std::fread(h, 1, 512, f) == 512 && h[0] != 0) {
        uint64_t size = 0;
        if (h[124] & 0x80) {
            for (int i = 125; i < 136; ++i) size = (size << 8) | h[i];
        } else {
            for (int i = 124; i < 136 && h[i] >= '0' && h[i] <= '7'; ++i) size = size * 8 + (h[i] - '0');
        }
        r->members.push_back({std::string((const char*)h, strnlen((const char*)h, 100)), pos + 512, size});
        pos += 512 + ((size + 511) & ~uint64_t(511));
    }
    *out = r;
    return SSB_OK;
}

int ssb_ckpt_member_count(const SsbCkptReader* r) { return r ? int(r->members.size()) : SSB_ERR_INVALID_ARGUMENT; }

int ssb_ckpt_member_info(const SsbCkptReader* r, int index, char* name, int name_capacity, uint64_t* size) {
    if (!r || index < 0 || index >= int(r->members.size())) return SSB_ERR_INVALID_ARGUMENT;
    const Member& m = r->members[index];
    if (name) {
        if (name_capacity <= int(m.name.size())) return SSB_ERR_CAPACITY;
        std::memcpy(name, m.name.c_str(), m.name.size() + 1);
    }
    if (size) *size = m.size;
    return SSB_OK;
}

int ssb_ckpt_read_bytes(SsbCkptReader* r, const char* name, void* buf, uint64_t capacity, uint64_t* size) {
    if (!r || !name) return SSB_ERR_INVALID_ARGUMENT;
    const Member* m = r->find(name);
    if (!m) return fail(SSB_ERR_INVALID_ARGUMENT, "checkpoint: no member '%s'", name);
    if (size) *size = m->size;
    if (!buf) return SSB_OK;
    if (capacity < m->size) return SSB_ERR_CAPACITY;
    if (!seek_to(r->f, m->offset) || std::fread(buf, 1, size_t(m->size), r->f) != m->size) return SSB_ERR_IO;
    return SSB_OK;
}

int ssb_ckpt_array_info(SsbCkptReader* r, const char* name, char* descr, int descr_capacity, uint64_t* data_bytes) {
    if (!r || !name) return SSB_ERR_INVALID_ARGUMENT;
    const Member* m = r->find(name);
    if (!m) return fail(SSB_ERR_INVALID_ARGUMENT, "checkpoint: no member '%s'", name);
    uint64_t off, bytes;
    std::string d;
    if (int rc = locate_array(r, *m, &off, &bytes, &d)) return rc;
    if (descr) {
        if (descr_capacity <= int(d.size())) return SSB_ERR_CAPACITY;
        std::memcpy(descr, d.c_str(), d.size() + 1);
    }
    if (data_bytes) *data_bytes = bytes;
    return SSB_OK;
}

int ssb_ckpt_read_host(SsbCkptReader* r, const char* name, void* h_ptr, uint64_t nbytes) {
    if (!r || !name || (!h_ptr && nbytes)) return SSB_ERR_INVALID_ARGUMENT;
    const Member* m = r->find(name);
    if (!m) return fail(SSB_ERR_INVALID_ARGUMENT, "checkpoint: no member '%s'", name);
    uint64_t off, bytes;
    std::string d;
    if (int rc = locate_array(r, *m, &off, &bytes, &d)) return rc;
    if (bytes != nbytes)
        return fail(SSB_ERR_CAPACITY, "checkpoint: size mismatch for '%s': file %llu vs buffer %llu", name,
                    (unsigned long long)bytes, (unsigned long long)nbytes);
    if (!seek_to(r->f, off) || std::fread(h_ptr, 1, size_t(nbytes), r->f) != nbytes) return SSB_ERR_IO;
    return SSB_OK;
}

int ssb_ckpt_read_device(SsbCkptReader* r, const char* name, void* d_ptr, uint64_t nbytes, void* stream) {
    if (!r || !name || (!d_ptr && nbytes)) return SSB_ERR_INVALID_ARGUMENT;
    const Member* m = r->find(name);
    if (!m) return fail(SSB_ERR_INVALID_ARGUMENT, "checkpoint: no member '%s'", name);
    uint64_t off, bytes;
    std::string d;
    if (int rc = locate_array(r, *m, &off, &bytes, &d)) return rc;
    if (bytes != nbytes)   // the reference refuses a slot whose byte size differs
        return fail(SSB_ERR_CAPACITY, "checkpoint: size mismatch for '%s': file %llu vs buffer %llu", name,
                    (unsigned long long)bytes, (unsigned long long)nbytes);
    if (int rc = r->stage.ensure()) return rc;
    if (!seek_to(r->f, off)) return SSB_ERR_IO;
    cudaStream_t st = (cudaStream_t)stream;
    char* dst = (char*)d_ptr;
    int rc = SSB_OK;
    bool used[2] = {false, false};
    for (uint64_t k = 0, done = 0; done < nbytes && rc == SSB_OK; ++k) {
        const size_t n = size_t(std::min<uint64_t>(kChunk, nbytes - done));
        const int b = int(k & 1);
        if (used[b] && cudaEventSynchronize(r->stage.done[b]) != cudaSuccess) rc = SSB_ERR_CUDA;   // buffer b is free again
        else if (std::fread(r->stage.buf[b], 1, n, r->f) != n) rc = SSB_ERR_IO;
        else if (cudaMemcpyAsync(dst + done, r->stage.buf[b], n, cudaMemcpyHostToDevice, st) != cudaSuccess ||
                 cudaEventRecord(r->stage.done[b], st) != cudaSuccess) rc = SSB_ERR_CUDA;
        used[b] = true;
        done += n;
    }
    if (cudaStreamSynchronize(st) != cudaSuccess && rc == SSB_OK) rc = SSB_ERR_CUDA;
    if (rc == SSB_ERR_CUDA) cudaGetLastError();
    return rc;
}

int ssb_ckpt_reader_close(SsbCkptReader* r) {
    if (!r) return SSB_ERR_INVALID_ARGUMENT;
    std::fclose(r->f);
    r->stage.release();
    delete r;
    return SSB_OK;
}

}  // extern "C"
