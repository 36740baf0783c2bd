// TEST INFRASTRUCTURE.  Calls the reference's own checkpoint container helpers
// (src/core/CheckpointIO.h) so that tests can compare the library's state.tar
// bytes with the reference's and hand the library's files to the reference's reader.
#include <fstream>
#include <sstream>
#include <cstring>
#include "core/CheckpointIO.h"

extern "C" {

// The NPY header the reference writes for a flat array; returns its length (or -1 if it does not fit).
int ref_ckpt_npy_header(const char* descr, uint64_t numel, char* out, int capacity) {
    std::string h = ckpt::npy_header(descr, (size_t)numel);
    if ((int)h.size() > capacity) return -1;
    std::memcpy(out, h.data(), h.size());
    return (int)h.size();
}

// One 512-byte member header as the reference writes it.
int ref_ckpt_tar_header(const char* name, uint64_t size, char* out512) {
    std::ostringstream o;
    ckpt::tar_header(o, name, (size_t)size);
    std::string s = o.str();
    if (s.size() != 512) return -1;
    std::memcpy(out512, s.data(), 512);
    return 0;
}

// A whole archive: state.json, then one array per entry.  With on_device != 0 the arrays are device
// buffers and go through tar_write_npy_device; otherwise they are host buffers and the same member
// is put together from npy_header + tar_write_bytes (the functions tar_write_npy_device is made of).
int ref_ckpt_write(const char* path, const char* json, int n, const char* const* names, const void* const* ptrs,
                   const uint64_t* nbytes, const uint8_t* tags, int on_device) {
    std::ofstream tar(path, std::ios::binary | std::ios::trunc);
    if (!tar) return -1;
    ckpt::tar_write_bytes(tar, "state.json", json, std::strlen(json));
    std::vector<char> stage;
    for (int i = 0; i < n; ++i) {
        std::string member = std::string(names[i]) + ".npy";
        if (on_device) {
            ckpt::tar_write_npy_device(tar, member, ptrs[i], (size_t)nbytes[i], tags[i], stage);
        } else {
            auto ds = npy_scalar_descr((NpyScalar)tags[i]);
            std::string blob = ckpt::npy_header(ds.first, (size_t)nbytes[i] / ds.second);
            blob.append((const char*)ptrs[i], (size_t)nbytes[i]);
            ckpt::tar_write_bytes(tar, member, blob.data(), blob.size());
        }
    }
    ckpt::tar_finish(tar);
    return tar.good() ? 0 : -1;
}

// The reference's load path for one member: index the archive, locate the array, check the byte size and
// copy it into device memory.  Returns 0, -1 (cannot open), -2 (no such member), -3 (size mismatch).
int ref_ckpt_read_device(const char* path, const char* name, void* d_ptr, uint64_t nbytes, char* descr8) {
    std::ifstream in(path, std::ios::binary);
    if (!in) return -1;
    std::string member = std::string(name) + ".npy";
    for (auto& m : ckpt::tar_index(in)) {
        if (m.name != member) continue;
        auto info = ckpt::npy_locate(in, m.data_offset, m.size);
        if (descr8) std::snprintf(descr8, 8, "%s", info.descr.c_str());
        if (info.data_bytes != nbytes) return -3;
        std::vector<char> stage;
        ckpt::read_into_device(in, info.data_offset, d_ptr, (size_t)nbytes, stage);
        return 0;
    }
    return -2;
}

// state.json as the reference's reader extracts it; returns its length or a negative code.
int ref_ckpt_read_json(const char* path, char* out, int capacity) {
    std::ifstream in(path, std::ios::binary);
    if (!in) return -1;
    for (auto& m : ckpt::tar_index(in)) {
        if (m.name != "state.json") continue;
        std::string s = ckpt::tar_read_member(in, m);
        if ((int)s.size() >= capacity) return -3;
        std::memcpy(out, s.data(), s.size());
        out[s.size()] = 0;
        return (int)s.size();
    }
    return -2;
}

}  // extern "C"
