// TEST INFRASTRUCTURE.  Helpers to hand raw device pointers to the reference's
// buffer views (src/primitives/PrimitiveBase3DGS.cuh:87-225).
#pragma once
#include "primitives/Primitive3DGS.cuh"

typedef Vanilla3DGS<3> RefPrim;

struct RawWorld : RefPrim::WorldBuffer {
    RawWorld(int64_t n, float* means, float* quats, float* scales, float* opacities, float* dc, float* sh) {
        _size = n;
        float* p[6] = {means, quats, scales, opacities, dc, sh};
        int32_t st[6] = {3, 4, 3, 1, 3, 45};
        for (int i = 0; i < 6; ++i) { _data[i] = p[i]; _strides[i] = st[i]; }
    }
};

struct RawScreen : RefPrim::ScreenBuffer {
    RawScreen(int64_t n, float* xy, float* depth, float* conic, float* opac, float* rgb) {
        _size = n;
        float* p[5] = {xy, depth, conic, opac, rgb};
        int32_t st[5] = {2, 1, 3, 1, 3};
        for (int i = 0; i < 5; ++i) { _data[i] = p[i]; _strides[i] = st[i]; }
    }
};
