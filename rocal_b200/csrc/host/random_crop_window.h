// Random-resized-crop windows of the fused JPEG crop source (rocalFusedJpegCrop[SingleShard]; the
// decoders.image_slice / image_random_crop calls of the Python API).
//
// The window of one image is a function of (height, width, 32-bit sample seed): the sample seed starts a
// std::mt19937, up to num_attempts (area, aspect) draws look for a window that fits, a clamped fallback follows,
// and the position is drawn last (rocAL/source/parameters/parameter_random_crop_decoder.cpp:41-96). The n sample
// seeds of a batch are std::seed_seq{batch seed}.generate() (same file, lines 104-108).
//
// The reference takes the batch seed from std::random_device, so its windows differ from run to run; here the
// batch seeds are the output sequence of a std::mt19937 started from the context's seed, which makes a run
// repeatable while every window is still one the reference can produce.
#pragma once
#include <cstddef>
#include <cstdint>
#include <random>
#include <vector>

namespace rb200 {

struct CropRect {
    unsigned x = 0, y = 0, w = 1, h = 1;
};

struct RandomCropRanges {
    float aspect_lo = 3.0f / 4, aspect_hi = 4.0f / 3;   // width / height
    float area_lo = 0.08f, area_hi = 1.0f;              // fraction of the image area
    int num_attempts = 10;
};

// The window for one image and one sample seed.
CropRect random_crop_window(int height, int width, uint32_t sample_seed, const RandomCropRanges& r);

// The n sample seeds that belong to one batch seed.
std::vector<uint32_t> random_crop_sample_seeds(uint32_t batch_seed, size_t n);

class RandomCropWindowSampler {
   public:
    RandomCropWindowSampler(const RandomCropRanges& r, uint32_t seed) : _ranges(r), _batch_seeds(seed) {}
    // Starts the next batch of n samples and returns its batch seed.
    uint32_t next_batch(size_t n);
    uint32_t batch_seed() const { return _batch_seed; }
    CropRect window(int height, int width, size_t sample) const;
    const RandomCropRanges& ranges() const { return _ranges; }

   private:
    RandomCropRanges _ranges;
    std::mt19937 _batch_seeds;
    uint32_t _batch_seed = 0;
    std::vector<uint32_t> _seeds;
};

}  // namespace rb200
