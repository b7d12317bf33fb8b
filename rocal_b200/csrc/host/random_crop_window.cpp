#include "random_crop_window.h"

#include <algorithm>
#include <cmath>

namespace rb200 {

namespace {

inline int at_least_one(int v) { return v < 1 ? 1 : v; }

}  // namespace

// Every intermediate below has the type the reference's expression gives it (int products before the
// conversion to float, float multiplies, float -> int truncation), because a window is only reproducible
// when each rounding happens in the same place.
CropRect random_crop_window(int height, int width, uint32_t sample_seed, const RandomCropRanges& r) {
    CropRect win;
    const int H = height, W = width;
    if (H <= 0 || W <= 0) return win;

    std::mt19937 gen(sample_seed);
    std::uniform_real_distribution<float> area_draw(r.area_lo, r.area_hi);
    std::uniform_real_distribution<float> log_aspect_draw(std::log(r.aspect_lo), std::log(r.aspect_hi));

    const float inv_aspect_lo = 1 / r.aspect_lo;                        // tallest allowed height / width
    const float least_area = (float)(W * H) * r.area_lo;
    const int widest = at_least_one((int)((float)H * r.aspect_hi));     // widest window of full height
    const int tallest = at_least_one((int)((float)W * inv_aspect_lo));  // tallest window of full width

    int cw = 1, ch = 1;
    if ((float)(H * widest) < least_area) {            // a very wide image: full height, widest allowed
        ch = H;
        cw = widest;
    } else if ((float)(W * tallest) < least_area) {    // a very tall image: full width, tallest allowed
        ch = tallest;
        cw = W;
    } else {
        bool found = false;
        for (int left = r.num_attempts; left > 0 && !found; left--) {
            const float frac = area_draw(gen);
            const float want = frac * (float)(size_t)(H * W);
            const float aspect = std::exp(log_aspect_draw(gen));
            cw = at_least_one((int)std::roundf(sqrtf(want * aspect)));
            ch = at_least_one((int)std::roundf(sqrtf(want / aspect)));
            const float got = (float)cw / (float)ch;
            found = cw <= W && ch <= H && got >= r.aspect_lo && got <= r.aspect_hi;
        }
        if (!found) {
            // no draw fitted: the whole image clamped to the aspect range, then shrunk to the largest area
            const float most_area = r.area_hi * (float)W * (float)H;
            const float whole = (float)W / (float)H;
            if (whole > r.aspect_hi) {
                ch = H;
                cw = widest;
            } else if (whole < r.aspect_lo) {
                ch = tallest;
                cw = W;
            } else {
                ch = H;
                cw = W;
            }
            const float shrink = std::min(1.0f, most_area / (float)((unsigned)cw * (unsigned)ch));
            const float side = std::sqrt(shrink);
            cw = at_least_one((int)((float)(unsigned)cw * side));
            ch = at_least_one((int)((float)(unsigned)ch * side));
        }
    }
    cw = std::min(cw, W);
    ch = std::min(ch, H);
    win.w = (unsigned)cw;
    win.h = (unsigned)ch;
    win.x = (unsigned)std::uniform_int_distribution<int>(0, W - cw)(gen);
    win.y = (unsigned)std::uniform_int_distribution<int>(0, H - ch)(gen);
    return win;
}

std::vector<uint32_t> random_crop_sample_seeds(uint32_t batch_seed, size_t n) {
    std::vector<uint32_t> seeds(n);
    std::seed_seq seq{batch_seed};
    seq.generate(seeds.begin(), seeds.end());
    return seeds;
}

uint32_t RandomCropWindowSampler::next_batch(size_t n) {
    _batch_seed = (uint32_t)_batch_seeds();
    _seeds = random_crop_sample_seeds(_batch_seed, n);
    return _batch_seed;
}

CropRect RandomCropWindowSampler::window(int height, int width, size_t sample) const {
    return random_crop_window(height, width, _seeds.at(sample), _ranges);
}

}  // namespace rb200
