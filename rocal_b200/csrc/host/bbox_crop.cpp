#include "bbox_crop.h"

#include <algorithm>
#include <cmath>

namespace rb200 {

BBoxCropSampler::BBoxCropSampler(uint32_t seed, bool all_boxes_overlap, bool has_shape)
    : _all_boxes_overlap(all_boxes_overlap), _has_shape(has_shape) {
    std::mt19937 master(seed);
    _rngs.reserve(128);
    for (int k = 0; k < 128; k++) {
        uint32_t w[4];
        for (auto& v : w) v = (uint32_t)master();
        std::seed_seq seq(w, w + 4);
        _rngs.emplace_back(seq);
    }
}

// intersection over union in float, as the reference evaluates it for this sampler (its is_iou branch)
static float iou_ltrb(const float* box, const float* crop) {
    const float xa = std::max(box[0], crop[0]), ya = std::max(box[1], crop[1]);
    const float xb = std::min(box[2], crop[2]), yb = std::min(box[3], crop[3]);
    const float inter = std::max(0.0f, xb - xa) * std::max(0.0f, yb - ya);
    const float a1 = (box[3] - box[1]) * (box[2] - box[0]);
    const float a2 = (crop[3] - crop[1]) * (crop[2] - crop[0]);
    return inter / float(a1 + a2 - inter);
}

void BBoxCropSampler::window(const float* boxes, int nb, int img_width, float out[4]) {
    static const float kOptions[7] = {-1.0f, 0.1f, 0.3f, 0.5f, 0.7f, 0.9f, 0.0f};
    std::mt19937& gen = _rngs[_count % _rngs.size()];
    _count++;
    std::uniform_int_distribution<> option_dis(0, 6);
    std::uniform_real_distribution<float> factor_dis(0.3, 1.0);
    float crop[4] = {0.f, 0.f, 1.f, 1.f};
    for (;;) {
        const int option = option_dis(gen);
        if (option == 6 || _has_shape) {
            crop[0] = crop[1] = 0.f;
            crop[2] = crop[3] = 1.f;
            break;
        }
        const float min_iou = kOptions[option];
        const float wf = factor_dis(gen), hf = factor_dis(gen);
        if ((wf / hf < 0.5) || (wf / hf > 2.)) continue;
        std::uniform_real_distribution<float> l_dis(0.0, 1.0 - wf), t_dis(0.0, 1.0 - hf);
        float x = l_dis(gen);
        const float y = t_dis(gen);
        x = (float)(std::lround(x * img_width) & ~7) / img_width;
        crop[0] = x; crop[1] = y; crop[2] = x + wf; crop[3] = y + hf;
        bool ok = true;
        if (_all_boxes_overlap)
            for (int j = 0; j < nb && ok; j++)
                if (iou_ltrb(boxes + 4 * j, crop) < min_iou) ok = false;
        if (!ok) continue;
        int inside = 0;
        for (int j = 0; j < nb; j++) {
            const double xc = 0.5 * (boxes[4 * j] + boxes[4 * j + 2]), yc = 0.5 * (boxes[4 * j + 1] + boxes[4 * j + 3]);
            if (xc > crop[0] && xc < crop[2] && yc > crop[1] && yc < crop[3]) inside++;
        }
        if (inside == 0) continue;
        break;
    }
    out[0] = crop[0];
    out[1] = crop[1];
    out[2] = crop[2] - crop[0];
    out[3] = crop[3] - crop[1];
}

}  // namespace rb200
