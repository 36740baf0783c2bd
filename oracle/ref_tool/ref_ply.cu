// TEST INFRASTRUCTURE.  The reference's splat.ply reader (src/checkpoint/SplatPly.cpp:159-254), compiled from its own
// source file, behind two C entry points: the vertex count and SH degree of a file, and its arrays copied into caller
// buffers (sized from the first call).  Returns 0, 1 when the reader says the file is not a splat PLY, 2 when it throws.
#include "checkpoint/SplatPly.cpp"

#include <cstring>

extern "C" int ref_ply_info(const char* path, int64_t* num, int* sh_degree) {
    try {
        if (!spirula::is_splat_ply(path)) return 1;
        const spirula::SplatCloud c = spirula::read_splat_ply(path, true);
        *num = c.num;
        *sh_degree = c.sh_degree;
        return 0;
    } catch (const std::exception&) {
        return 2;
    }
}

extern "C" int ref_ply_read(const char* path, float* means, float* quats, float* scales, float* opacities, float* features_dc, float* features_sh) {
    try {
        const spirula::SplatCloud c = spirula::read_splat_ply(path, features_sh != nullptr);
        std::memcpy(means, c.means.data(), c.means.size() * sizeof(float));
        std::memcpy(quats, c.quats.data(), c.quats.size() * sizeof(float));
        std::memcpy(scales, c.scales.data(), c.scales.size() * sizeof(float));
        std::memcpy(opacities, c.opacities.data(), c.opacities.size() * sizeof(float));
        std::memcpy(features_dc, c.features_dc.data(), c.features_dc.size() * sizeof(float));
        if (features_sh) std::memcpy(features_sh, c.features_sh.data(), c.features_sh.size() * sizeof(float));
        return 0;
    } catch (const std::exception&) {
        return 2;
    }
}
