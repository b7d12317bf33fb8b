/*
 * ref_bbox_crop_driver.cpp — C entry point around the reference's random-bbox-crop sampler. TEST INFRASTRUCTURE ONLY.
 *
 * Built by oracle/build.py into oracle/_ref/libref.so together with
 * rocAL/source/meta_data/randombboxcrop_reader.cpp, compiled where it lies (nothing of the reference is copied).
 *
 *   ref_random_bbox_crop -> RandomBBoxCropReader::get_batch_crop_coords
 *                           (rocAL/source/meta_data/randombboxcrop_reader.cpp:216-313)
 *
 * The reader seeds its 128 generators from std::random_device, so its windows differ from run to run. To compare a
 * restatement with it, this driver replaces the generators by ones of a stated seeding (the class keeps them private:
 * the header is read with `private` spelled `public`, which does not change the layout): a std::mt19937 started from
 * `seed` hands out four words per generator, which seed it through std::seed_seq - the reader's own scheme
 * (SeededRNG<std::mt19937, 4>, include/meta_data/randombboxcrop_reader.h:41-72) with the random_device words replaced.
 * Boxes reach the sampler through a MetaDataReader stand-in that serves one BoundingBox record per image name.
 */
#include <algorithm>
#include <array>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <functional>
#include <iomanip>
#include <iostream>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <numeric>
#include <queue>
#include <random>
#include <set>
#include <sstream>
#include <string>
#include <thread>
#include <tuple>
#include <unordered_map>
#include <variant>
#include <vector>

// every standard header is in by now (their guards keep the next line away from the library's own classes)
#define private public
#include "meta_data/randombboxcrop_reader.h"
#undef private

namespace {
class MapReader : public MetaDataReader {
   public:
    std::map<std::string, std::shared_ptr<MetaData>> content;
    void init(const MetaDataConfig&, pMetaDataBatch) override {}
    void read_all(const std::string&) override {}
    void lookup(const std::vector<std::string>&) override {}
    void release() override {}
    const std::map<std::string, std::shared_ptr<MetaData>>& get_map_content() override { return content; }
    bool exists(const std::string& name) override { return content.count(name) != 0; }
    bool set_timestamp_mode() override { return false; }
};
}  // namespace

/* boxes: [total][4] ltrb as the sampler should see them (normalized); box_offsets [n+1]; img_w [n] image widths in
 * pixels (the sampler aligns the window's left edge to 8 pixels); out_xywh [n][4]. */
extern "C" __attribute__((visibility("default"))) int ref_random_bbox_crop(const float* boxes, const int32_t* box_offsets, int n,
                                                                           const int32_t* img_w, unsigned seed, int all_boxes_overlap,
                                                                           float* out_xywh) {
    auto reader = std::make_shared<RandomBBoxCropReader>();
    RandomBBoxCrop_MetaDataConfig cfg(RandomBBoxCrop_MetaDataType::BoundingBox, RandomBBoxCrop_MetaDataReaderType::RandomBBoxCropReader,
                                      all_boxes_overlap != 0, /*no_crop*/ false, nullptr, /*has_shape*/ false, 0, 0, 1, nullptr, 0, 0);
    auto batch = std::make_shared<CropCordBatch>();
    reader->init(cfg, batch);
    std::mt19937 master(seed);
    for (size_t k = 0; k < reader->_rngs._rngs.size(); k++) {
        uint32_t w[4];
        for (auto& v : w) v = (uint32_t)master();
        std::seed_seq seq(w, w + 4);
        reader->_rngs._rngs[k] = std::mt19937(seq);
    }
    auto meta = std::make_shared<MapReader>();
    std::vector<std::string> names;
    for (int i = 0; i < n; i++) {
        BoundingBoxCords cords;
        Labels labels;
        for (int b = box_offsets[i]; b < box_offsets[i + 1]; b++) {
            cords.emplace_back(boxes[b * 4 + 0], boxes[b * 4 + 1], boxes[b * 4 + 2], boxes[b * 4 + 3]);
            labels.push_back(1);
        }
        const std::string name = std::to_string(i);
        meta->content[name] = std::make_shared<BoundingBox>(cords, labels, ImgSize{img_w[i], img_w[i]});
        names.push_back(name);
    }
    reader->set_meta_data(meta);
    auto coords = reader->get_batch_crop_coords(names);
    for (int i = 0; i < n; i++)
        for (int k = 0; k < 4; k++) out_xywh[i * 4 + k] = coords[i][k];
    return 0;
}
