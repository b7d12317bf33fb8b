// The host side of the pipeline (graph planning, loader thread, ring of output slots, feeding ahead, boxes, random
// bbox crop) driven through the rocAL-signature API on the stand-in runtime of fake_cuda_runtime.cpp. One thread feeds
// batches as fast as it can while the main thread runs and reads them, so that the thread sanitizer sees the
// producer / loader / consumer hand-offs and the address sanitizer every table and buffer the host code sizes.
// Batch k's images are filled with the value k, and the stand-in kernels write a sample's first source byte into its
// whole output, so the order and the lifetime of the batches can be checked: output k must read k everywhere.
//
//   harness <batches>      prints "ok <batches>" and exits 0
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "rb200.h"
#include "rocal_api.h"

#define CHECK(ctx, cond)                                                                               \
    do {                                                                                               \
        if (!(cond)) {                                                                                 \
            fprintf(stderr, "line %d: %s failed: %s\n", __LINE__, #cond, rocalGetErrorMessage(ctx));   \
            return 1;                                                                                  \
        }                                                                                              \
    } while (0)

int main(int argc, char** argv) {
    const int batches = argc > 1 ? atoi(argv[1]) : 40;
    const int n = 6, W = 40, H = 30;

    RocalContext ctx = rocalCreate((size_t)n, ROCAL_PROCESS_GPU, 0, 1, 3, ROCAL_FP32);
    if (!ctx) return 1;
    rocalSetSeed(5);
    RocalTensor src = rocalJpegExternalFileSource(ctx, ROCAL_COLOR_RGB24, false, false, false, ROCAL_USE_USER_GIVEN_SIZE, W, H,
                                                  ROCAL_DECODER_TJPEG, ROCAL_EXTSOURCE_RAW_UNCOMPRESSED);
    CHECK(ctx, src);
    rocalRandomBBoxCrop(ctx, false, true, NULL, false, 0, 0, 1, NULL, 0, 9);
    RocalTensor r = rocalResize(ctx, src, 16, 12, true, ROCAL_SCALING_MODE_STRETCH);
    CHECK(ctx, r);
    RocalTensor b = rocalBrightnessFixed(ctx, r, 1.0f, 0.0f, false);
    CHECK(ctx, b);
    std::vector<float> mean{0.f, 0.f, 0.f}, sd{1.f, 1.f, 1.f};
    RocalIntParam coin = rocalCreateIntUniformRand(0, 1);
    RocalTensor o = rocalCropMirrorNormalize(ctx, b, 8, 8, 0.5f, 0.5f, mean, sd, true, coin, ROCAL_NCHW, ROCAL_FP32);
    CHECK(ctx, o);
    std::vector<float> anchors;
    for (int i = 0; i < 32; i++) { anchors.insert(anchors.end(), {0.03f * i, 0.02f * i, 0.03f * i + 0.1f, 0.02f * i + 0.2f}); }
    std::vector<float> means{0.f, 0.f, 0.f, 0.f}, stds{0.1f, 0.1f, 0.2f, 0.2f};
    rocalBoxEncoder(ctx, anchors, 0.5f, means, stds, true, 1.0f);
    CHECK(ctx, rb200_set_profiling(ctx, 1) == 0);
    CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);

    // every batch keeps its own host buffers until the end: the pipeline may read them until the batch is returned
    std::vector<std::vector<unsigned char>> arenas((size_t)batches, std::vector<unsigned char>((size_t)n * W * H * 3 + 256));
    std::vector<rb200_image_desc> descs((size_t)n);
    for (int i = 0; i < n; i++) descs[(size_t)i] = {(uint64_t)i * W * H * 3, (uint32_t)W * 3, (uint32_t)W, (uint32_t)H};
    std::atomic<int> fed{0};
    std::atomic<int> feed_failed{0};
    std::thread producer([&] {
        for (int k = 0; k < batches; k++) {
            std::memset(arenas[(size_t)k].data(), k & 0xFF, arenas[(size_t)k].size());
            std::vector<float> boxes;
            std::vector<int> labels, counts;
            for (int i = 0; i < n; i++) {
                const int c = 1 + (i + k) % 3;
                counts.push_back(c);
                for (int j = 0; j < c; j++) {
                    boxes.insert(boxes.end(), {0.1f + 0.05f * j, 0.2f, 0.6f + 0.05f * j, 0.9f});
                    labels.push_back(1 + j);
                }
            }
            if (rb200_feed_boxes(ctx, boxes.data(), labels.data(), counts.data(), (size_t)n) != 0 ||
                rb200_feed_ragged(ctx, arenas[(size_t)k].data(), arenas[(size_t)k].size(), descs.data(), (size_t)n, RB200_MEM_HOST) != 0) {
                feed_failed = 1;
                return;
            }
            fed++;
        }
    });

    std::vector<unsigned char> host_r((size_t)n * 12 * 16 * 3);
    std::vector<float> host_o((size_t)n * 3 * 8 * 8);
    std::vector<float> enc((size_t)n * 32 * 4);
    std::vector<int> enc_labels((size_t)n * 32);
    for (int k = 0; k < batches; k++) {
        while (fed.load() <= k && !feed_failed.load()) std::this_thread::yield();
        CHECK(ctx, !feed_failed.load());
        CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
        RocalTensorList tl = rocalGetOutputTensors(ctx);
        CHECK(ctx, tl && tl->size() == 2);
        CHECK(ctx, tl->at(0)->copy_data(host_r.data(), ROCAL_MEMCPY_HOST) == 0);
        CHECK(ctx, tl->at(1)->copy_data(host_o.data(), ROCAL_MEMCPY_HOST) == 0);
        for (unsigned char v : host_r) CHECK(ctx, v == (unsigned char)(k & 0xFF));
        for (float v : host_o) CHECK(ctx, v == (float)(k & 0xFF));
        std::vector<float> gb(64 * 4);
        std::vector<int> gl(64), gc((size_t)n);
        const size_t total = rb200_get_bounding_boxes(ctx, gb.data(), gl.data(), gc.data());
        CHECK(ctx, total >= (size_t)n && total <= 64);
        rocalCopyEncodedBoxesAndLables(ctx, enc.data(), enc_labels.data());
        for (int i = 0; i < n; i++) CHECK(ctx, enc_labels[(size_t)i * 32] == gc[(size_t)i]);    // the encoder saw this batch's boxes
        int coins[6];          // the returned batch's own draws, read while the loader prepares later batches
        CHECK(ctx, rb200_get_batch_int_array(ctx, coin, coins, 6) == 6);
        for (int i = 0; i < n; i++) CHECK(ctx, coins[i] == 0 || coins[i] == 1);
        unsigned win[6 * 4];
        CHECK(ctx, rb200_get_decoder_crop_windows(ctx, win, nullptr) == 0);
        for (int i = 0; i < n; i++) CHECK(ctx, win[i * 4] + win[i * 4 + 2] <= (unsigned)W && win[i * 4 + 1] + win[i * 4 + 3] <= (unsigned)H);
    }
    producer.join();
    CHECK(ctx, rocalGetStatus(ctx) == ROCAL_OK);
    rb200_step_timing st[8];
    const size_t steps = rb200_get_step_timing(ctx, st, 8);
    CHECK(ctx, steps == 4 && std::strcmp(st[0].name, "upload") == 0 && std::strcmp(st[1].name, "resample") == 0);
    for (size_t i = 0; i < steps; i++) CHECK(ctx, st[i].batches == (unsigned long long)batches && st[i].gpu_us > 0.0);
    // nothing left to run: the call fails with a message and the context stays usable
    CHECK(ctx, rocalRun(ctx) != ROCAL_OK);
    CHECK(ctx, std::strstr(rocalGetErrorMessage(ctx), "no input batch") != nullptr);
    // a batch without boxes is refused by the box-aware crop when its turn comes, and reported by rocalRun
    CHECK(ctx, rb200_feed_ragged(ctx, arenas[0].data(), arenas[0].size(), descs.data(), (size_t)n, RB200_MEM_HOST) == 0);
    CHECK(ctx, rocalRun(ctx) != ROCAL_OK);
    CHECK(ctx, std::strstr(rocalGetErrorMessage(ctx), "no bounding boxes") != nullptr);
    // release with batches still queued and in flight: the loader thread is stopped and joined first
    for (int k = 0; k < 3 && k < batches; k++) {
        std::vector<float> boxes{0.1f, 0.1f, 0.9f, 0.9f, 0.1f, 0.1f, 0.9f, 0.9f, 0.1f, 0.1f, 0.9f, 0.9f,
                                 0.1f, 0.1f, 0.9f, 0.9f, 0.1f, 0.1f, 0.9f, 0.9f, 0.1f, 0.1f, 0.9f, 0.9f};
        std::vector<int> labels(6, 1), counts(6, 1);
        CHECK(ctx, rb200_feed_boxes(ctx, boxes.data(), labels.data(), counts.data(), (size_t)n) == 0);
        CHECK(ctx, rb200_feed_ragged(ctx, arenas[(size_t)k].data(), arenas[(size_t)k].size(), descs.data(), (size_t)n, RB200_MEM_HOST) == 0);
    }
    CHECK(ctx, rb200_set_profiling(ctx, 0) != 0);      // too late: the events are part of the plan
    TimingInfo t = rocalGetTimingInfo(ctx);
    (void)t;
    rocalRelease(ctx);
    printf("ok %d\n", batches);
    return 0;
}
