// Random bounding-box crop windows (rocalRandomBBoxCrop; fn.random_bbox_crop of the Python API).
//
// Per sample, from that sample position's own std::mt19937 (128 of them serve the samples in turn, as the reference's
// SeededRNG<std::mt19937, 4>, rocAL/include/meta_data/randombboxcrop_reader.h:41-72): one of seven minimum-IoU options
// {-1, 0.1, 0.3, 0.5, 0.7, 0.9, keep the whole image}, a width and a height factor in 0.3 .. 1 whose ratio lies in
// 0.5 .. 2, a position with the left edge aligned to 8 pixels; with all_boxes_overlap every box must reach the
// option's IoU with the window; at least one box centre must lie strictly inside. A draw that fails any test starts
// over (RandomBBoxCropReader::get_batch_crop_coords, rocAL/source/meta_data/randombboxcrop_reader.cpp:216-313).
//
// The reference seeds its generators from std::random_device; here generator k is seeded through std::seed_seq from
// outputs 4k .. 4k+3 of a std::mt19937 started from the given seed, so a run is repeatable and every window is one
// the reference can produce.
#pragma once
#include <cstddef>
#include <cstdint>
#include <random>
#include <vector>

namespace rb200 {

class BBoxCropSampler {
   public:
    BBoxCropSampler(uint32_t seed, bool all_boxes_overlap, bool has_shape);
    // boxes: nb x {l, t, r, b} normalized to the image; out: {x, y, w, h} normalized
    void window(const float* boxes, int nb, int img_width, float out[4]);

   private:
    std::vector<std::mt19937> _rngs;
    size_t _count = 0;
    bool _all_boxes_overlap, _has_shape;
};

}  // namespace rb200
