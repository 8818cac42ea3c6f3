// C entry points around the reference's own src/modules/preprocess.h (included from the reference tree at build
// time, never copied), so that tests can hold the oracle's restatement of the image preprocessing and of the
// pixel-shuffle order against the reference's code itself.  Test infrastructure only.
#include <cstdint>
#include <cstring>
#include <vector>

#include "modules/preprocess.h"

extern "C" {

// pixels: side * side * 3 (H, W, C), uint8 or float32; out: 3 * side * side floats (C, H, W).  Returns 1 on success.
int ref_preprocess_image_chw(const void *pixels, int is_f32, int side, float *out) {
    vla::ImageView v{pixels, side, side, is_f32 ? vla::PixelFormat::F32_RGB_01 : vla::PixelFormat::U8};
    std::vector<float> chw;
    if (!vla::preprocess_image_chw("shim", v, side, chw)) return 0;
    std::memcpy(out, chw.data(), chw.size() * sizeof(float));
    return 1;
}

// src: [n_patches][embed]; dst: [(grid / s)^2][embed * s * s]
void ref_pixel_shuffle_hf(const float *src, float *dst, int64_t embed, int64_t grid, int64_t s) {
    vla::pixel_shuffle_hf(src, dst, embed, grid, s);
}

}
