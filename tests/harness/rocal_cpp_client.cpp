// A C++ application written against the rocAL-signature header (include/rocal_api.h), in the style of the
// reference's tests/cpp_api/unit_tests/unit_tests.cpp: it builds two graphs with the reference's call sequence,
// feeds images from a binary file and writes every result to another one. tests/test_cpp_client_gpu.py compiles
// it with g++ (no CUDA headers needed), runs it and checks the results against the oracle.
//
//   client <in.bin> <out.bin> [jpeg_folder]
// in.bin : int32 n, then n x {int32 h, int32 w}, then the n images (uint8 HWC, tightly packed),
//          then int32 total_boxes, n x int32 counts, total x 4 float32 ltrb, total x int32 labels,
//          then int32 num_anchors, num_anchors x 4 float32
// out.bin: graph 1 output (n x 3 x 224 x 224 float32), n x int32 mirror flags read back per run is not possible from
//          C++, so graph 1 uses mirror = 0; graph 2 output (n x 3 x 300 x 300 float32), int32 box count,
//          per sample int32 count + boxes + labels, encoded boxes (n x A x 4 float32) and labels (n x A int32).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "rb200.h"
#include "rocal_api.h"

static std::vector<unsigned char> slurp(const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", path); exit(2); }
    fseek(f, 0, SEEK_END);
    long len = ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<unsigned char> d((size_t)len);
    if (fread(d.data(), 1, (size_t)len, f) != (size_t)len) exit(2);
    fclose(f);
    return d;
}

#define CHECK(ctx, cond)                                                                      \
    do {                                                                                      \
        if (!(cond)) {                                                                        \
            fprintf(stderr, "line %d: %s failed: %s\n", __LINE__, #cond, rocalGetErrorMessage(ctx)); \
            return 1;                                                                         \
        }                                                                                     \
    } while (0)

int main(int argc, char** argv) {
    if (argc < 3 || argc > 5) return 2;
    std::vector<unsigned char> in = slurp(argv[1]);
    const unsigned char* p = in.data();
    auto rd_i32 = [&]() { int v; memcpy(&v, p, 4); p += 4; return v; };
    const int n = rd_i32();
    std::vector<int> hs(n), ws(n);
    int max_h = 0, max_w = 0;
    for (int i = 0; i < n; i++) { hs[i] = rd_i32(); ws[i] = rd_i32(); if (hs[i] > max_h) max_h = hs[i]; if (ws[i] > max_w) max_w = ws[i]; }
    // the reference's feed contract: one max-size slot per image, the valid region at its origin
    std::vector<std::vector<unsigned char>> slots(n, std::vector<unsigned char>((size_t)max_h * max_w * 3, 0));
    std::vector<unsigned char*> bufs(n);
    std::vector<ROIxywh> rois(n);
    for (int i = 0; i < n; i++) {
        for (int y = 0; y < hs[i]; y++) memcpy(&slots[i][(size_t)y * max_w * 3], p + (size_t)y * ws[i] * 3, (size_t)ws[i] * 3);
        p += (size_t)hs[i] * ws[i] * 3;
        bufs[i] = slots[i].data();
        rois[i] = {0, 0, (unsigned)ws[i], (unsigned)hs[i]};
    }
    const int total = rd_i32();
    std::vector<int> counts(n);
    for (int i = 0; i < n; i++) counts[i] = rd_i32();
    std::vector<float> boxes((size_t)total * 4);
    memcpy(boxes.data(), p, boxes.size() * 4); p += boxes.size() * 4;
    std::vector<int> labels(total);
    memcpy(labels.data(), p, (size_t)total * 4); p += (size_t)total * 4;
    const int A = rd_i32();
    std::vector<float> anchors((size_t)A * 4);
    memcpy(anchors.data(), p, anchors.size() * 4);

    FILE* out = fopen(argv[2], "wb");
    if (!out) return 2;
    std::vector<float> mean{123.675f, 116.28f, 103.53f}, sd{58.395f, 57.12f, 57.375f};

    // ---- graph 1: Resize(shorter 256) -> CropMirrorNormalize 224 (centre crop, no mirror), fp32 NCHW ----
    {
        RocalContext ctx = rocalCreate((size_t)n, ROCAL_PROCESS_GPU, 0, 1, 2, ROCAL_FP32);
        if (!ctx) return 1;
        RocalTensor src = rocalJpegExternalFileSource(ctx, ROCAL_COLOR_RGB24, false, false, false, ROCAL_USE_USER_GIVEN_SIZE,
                                                      (unsigned)max_w, (unsigned)max_h, ROCAL_DECODER_TJPEG, ROCAL_EXTSOURCE_RAW_UNCOMPRESSED);
        CHECK(ctx, src);
        RocalTensor r = rocalResize(ctx, src, 0, 0, false, ROCAL_SCALING_MODE_DEFAULT, {}, 256);
        CHECK(ctx, r);
        RocalIntParam mirror = rocalCreateIntParameter(0);
        RocalTensor o = rocalCropMirrorNormalize(ctx, r, 224, 224, 0.5f, 0.5f, mean, sd, true, mirror, ROCAL_NCHW, ROCAL_FP32);
        CHECK(ctx, o);
        CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);
        CHECK(ctx, rocalGetAugmentationBranchCount(ctx) == 1 && rocalGetOutputWidth(ctx) == 224);
        CHECK(ctx, rocalExternalSourceFeedInput(ctx, {}, false, bufs, rois, (unsigned)max_w, (unsigned)max_h, 3,
                                                ROCAL_EXTSOURCE_RAW_UNCOMPRESSED, ROCAL_NHWC, false) == ROCAL_OK);
        CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
        RocalTensorList tl = rocalGetOutputTensors(ctx);
        CHECK(ctx, tl && tl->size() == 1);
        rocalTensor* t = tl->at(0);
        CHECK(ctx, t->backend() == ROCAL_GPU && t->data_type() == ROCAL_FP32 && t->dims()[1] == 3 && t->dims()[3] == 224);
        std::vector<float> host(t->data_size() / 4);
        CHECK(ctx, t->copy_data(host.data(), ROCAL_MEMCPY_HOST) == 0);
        fwrite(host.data(), 4, host.size(), out);
        CHECK(ctx, rocalGetStatus(ctx) == ROCAL_OK);
        rocalRelease(ctx);
    }
    // ---- graph 2: SSDRandomCrop -> Resize 300x300 -> CropMirrorNormalize + BoxEncoder ----
    {
        RocalContext ctx = rocalCreate((size_t)n, ROCAL_PROCESS_GPU, 0, 1, 2, ROCAL_FP32);
        if (!ctx) return 1;
        rocalSetSeed(77);
        RocalTensor src = rocalJpegExternalFileSource(ctx, ROCAL_COLOR_RGB24, false, false, false, ROCAL_USE_USER_GIVEN_SIZE,
                                                      (unsigned)max_w, (unsigned)max_h, ROCAL_DECODER_TJPEG, ROCAL_EXTSOURCE_RAW_UNCOMPRESSED);
        CHECK(ctx, src);
        RocalTensor c = rocalSSDRandomCrop(ctx, src, false);
        CHECK(ctx, c);
        RocalTensor r = rocalResize(ctx, c, 300, 300, false, ROCAL_SCALING_MODE_STRETCH);
        CHECK(ctx, r);
        RocalTensor o = rocalCropMirrorNormalize(ctx, r, 300, 300, 0.f, 0.f, mean, sd, true, rocalCreateIntParameter(0), ROCAL_NCHW, ROCAL_FP32);
        CHECK(ctx, o);
        std::vector<float> means{0.f, 0.f, 0.f, 0.f}, stds{0.1f, 0.1f, 0.2f, 0.2f};
        rocalBoxEncoder(ctx, anchors, 0.5f, means, stds, true, 1.0f);
        CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);
        CHECK(ctx, rb200_feed_boxes(ctx, boxes.data(), labels.data(), counts.data(), (size_t)n) == 0);
        CHECK(ctx, rocalExternalSourceFeedInput(ctx, {}, false, bufs, rois, (unsigned)max_w, (unsigned)max_h, 3,
                                                ROCAL_EXTSOURCE_RAW_UNCOMPRESSED, ROCAL_NHWC, false) == ROCAL_OK);
        CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
        rocalTensor* t = rocalGetOutputTensors(ctx)->at(0);
        std::vector<float> host(t->data_size() / 4);
        CHECK(ctx, t->copy_data(host.data(), ROCAL_MEMCPY_HOST) == 0);
        fwrite(host.data(), 4, host.size(), out);
        // crop windows (extension) so that the checker can rebuild the expected image
        std::vector<unsigned> win((size_t)n * 4);
        CHECK(ctx, rb200_get_crop_windows(ctx, c, win.data()) == 0);
        fwrite(win.data(), 4, win.size(), out);
        // boxes after the crop, through the reference's getters
        int bc = (int)rocalGetBoundingBoxCount(ctx);
        fwrite(&bc, 4, 1, out);
        RocalTensorList bl = rocalGetBoundingBoxCords(ctx), ll = rocalGetBoundingBoxLabel(ctx);
        CHECK(ctx, bl && ll && bl->size() == (uint64_t)n && ll->size() == (uint64_t)n);
        for (int i = 0; i < n; i++) {
            int cnt = (int)bl->at(i)->dims()[0];
            CHECK(ctx, bl->at(i)->backend() == ROCAL_CPU && (int)ll->at(i)->dims()[0] == cnt);
            fwrite(&cnt, 4, 1, out);
            std::vector<float> b((size_t)cnt * 4);
            std::vector<int> l(cnt);
            CHECK(ctx, bl->at(i)->copy_data(b.data(), ROCAL_MEMCPY_HOST) == 0 && ll->at(i)->copy_data(l.data(), ROCAL_MEMCPY_HOST) == 0);
            fwrite(b.data(), 4, b.size(), out);
            fwrite(l.data(), 4, l.size(), out);
        }
        std::vector<float> eb((size_t)n * A * 4);
        std::vector<int> el((size_t)n * A);
        rocalCopyEncodedBoxesAndLables(ctx, eb.data(), el.data());
        fwrite(eb.data(), 4, eb.size(), out);
        fwrite(el.data(), 4, el.size(), out);
        CHECK(ctx, rocalGetStatus(ctx) == ROCAL_OK);
        rocalRelease(ctx);
    }
    // ---- graph 3: CropResizeFixed, ROIResize (triangular), RandomCrop with fixed parameters, Copy ----
    {
        RocalContext ctx = rocalCreate((size_t)n, ROCAL_PROCESS_GPU, 0, 1, 2, ROCAL_FP32);
        if (!ctx) return 1;
        RocalTensor src = rocalJpegExternalFileSource(ctx, ROCAL_COLOR_RGB24, false, false, false, ROCAL_USE_USER_GIVEN_SIZE,
                                                      (unsigned)max_w, (unsigned)max_h, ROCAL_DECODER_TJPEG, ROCAL_EXTSOURCE_RAW_UNCOMPRESSED);
        CHECK(ctx, src);
        RocalTensor cr = rocalCropResizeFixed(ctx, src, 120, 80, true, 0.5f, 1.25f, 0.25f, 0.75f);
        CHECK(ctx, cr);
        RocalTensor roi = rocalROIResize(ctx, src, 64, 48, true, 100, 150, 20.f, 30.f, ROCAL_TRIANGULAR_INTERPOLATION);
        CHECK(ctx, roi);
        RocalTensor rc = rocalRandomCrop(ctx, src, true, rocalCreateFloatParameter(0.5f), rocalCreateFloatParameter(1.25f),
                                         rocalCreateFloatParameter(0.25f), rocalCreateFloatParameter(0.75f));
        CHECK(ctx, rc);
        RocalTensor cp = rocalCopy(ctx, src, true);
        CHECK(ctx, cp);
        CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);
        CHECK(ctx, rocalGetAugmentationBranchCount(ctx) == 4);
        CHECK(ctx, rocalExternalSourceFeedInput(ctx, {}, false, bufs, rois, (unsigned)max_w, (unsigned)max_h, 3,
                                                ROCAL_EXTSOURCE_RAW_UNCOMPRESSED, ROCAL_NHWC, false) == ROCAL_OK);
        CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
        RocalTensorList tl = rocalGetOutputTensors(ctx);
        CHECK(ctx, tl && tl->size() == 4);
        for (int k = 0; k < 4; k++) {
            rocalTensor* t = tl->at(k);
            CHECK(ctx, t->data_type() == ROCAL_UINT8 && t->layout() == ROCAL_NHWC);
            std::vector<unsigned char> host(t->data_size());
            CHECK(ctx, t->copy_data(host.data(), ROCAL_MEMCPY_HOST) == 0);
            const int dims[2] = {(int)t->dims()[1], (int)t->dims()[2]};     // height, width of the padded output
            fwrite(dims, 4, 2, out);
            fwrite(host.data(), 1, host.size(), out);
            std::vector<unsigned> r4((size_t)n * 4);
            t->copy_roi(r4.data());
            fwrite(r4.data(), 4, r4.size(), out);
        }
        std::vector<int> sizes((size_t)n * 2);
        rocalGetImageSizes(ctx, sizes.data());
        fwrite(sizes.data(), 4, sizes.size(), out);
        CHECK(ctx, rocalGetStatus(ctx) == ROCAL_OK);
        rocalRelease(ctx);
    }
    // ---- graph 4 (with a folder of JPEG files): rocalCreateLabelReader + rocalFusedJpegCropSingleShard -> Resize ----
    if (argc >= 4) {
        const int bs = 2;
        RocalContext ctx = rocalCreate((size_t)bs, ROCAL_PROCESS_GPU, 0, 1, 2, ROCAL_FP32);
        if (!ctx) return 1;
        rocalSetSeed(321);
        rocalCreateLabelReader(ctx, argv[3]);
        std::vector<float> area{0.08f, 1.0f}, aspect{0.75f, 1.33333f};
        RocalShardingInfo sharding(RocalLastBatchPolicy::ROCAL_LAST_BATCH_PARTIAL, true, true, -1);
        RocalTensor src = rocalFusedJpegCropSingleShard(ctx, argv[3], ROCAL_COLOR_RGB24, 0, 1, false, area, aspect, 100, false, false,
                                                        ROCAL_USE_USER_GIVEN_SIZE, 400, 400, sharding);
        CHECK(ctx, src);
        RocalTensor r = rocalResize(ctx, src, 64, 64, true, ROCAL_SCALING_MODE_STRETCH, {}, 0, 0, ROCAL_TRIANGULAR_INTERPOLATION);
        CHECK(ctx, r);
        CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);
        const int remaining = (int)rocalGetRemainingImages(ctx);
        fwrite(&remaining, 4, 1, out);
        int batches = 0;
        while (!rocalIsEmpty(ctx)) {
            CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
            batches++;
            std::vector<int> labels(bs), sizes(bs * 2), lens(bs);
            RocalTensorList ll = rocalGetImageLabels(ctx);
            CHECK(ctx, ll && ll->size() == (uint64_t)bs && ll->at(0)->backend() == ROCAL_CPU && ll->at(0)->data_type() == ROCAL_INT32);
            for (int i = 0; i < bs; i++) labels[i] = static_cast<int*>(ll->at(0)->buffer())[i];
            CHECK(ctx, *static_cast<int*>(ll->at(1)->buffer()) == labels[1]);
            rocalGetImageSizes(ctx, sizes.data());
            const unsigned total = rocalGetImageNameLen(ctx, lens.data());
            std::vector<char> names(total + 1, 0);
            rocalGetImageName(ctx, names.data());
            std::vector<unsigned> win(bs * 4);
            unsigned seed = 0;
            CHECK(ctx, rb200_get_decoder_crop_windows(ctx, win.data(), &seed) == 0);
            const int padded = (int)rocalGetLastBatchPaddedSize(ctx);
            fwrite(labels.data(), 4, bs, out);
            fwrite(sizes.data(), 4, bs * 2, out);
            fwrite(lens.data(), 4, bs, out);
            fwrite(&total, 4, 1, out);
            fwrite(names.data(), 1, total, out);
            fwrite(win.data(), 4, bs * 4, out);
            fwrite(&seed, 4, 1, out);
            fwrite(&padded, 4, 1, out);
            rocalTensor* t = rocalGetOutputTensors(ctx)->at(0);
            CHECK(ctx, t->dims()[1] == 64 && t->dims()[2] == 64 && t->data_type() == ROCAL_UINT8);
        }
        fwrite(&batches, 4, 1, out);
        CHECK(ctx, rocalGetStatus(ctx) == ROCAL_OK);
        rocalRelease(ctx);
    }
    // ---- graph 5 (folder + COCO annotation file): rocalCreateCOCOReader + rocalJpegCOCOFileSourcePartialSingleShard -> Resize ----
    if (argc >= 5) {
        const int bs = 2;
        RocalContext ctx = rocalCreate((size_t)bs, ROCAL_PROCESS_GPU, 0, 1, 2, ROCAL_FP32);
        if (!ctx) return 1;
        rocalSetSeed(99);
        rocalCreateCOCOReader(ctx, argv[4], true);
        std::vector<float> area{0.3f, 0.8f}, aspect{0.5f, 2.0f};
        RocalTensor src = rocalJpegCOCOFileSourcePartialSingleShard(ctx, argv[3], argv[4], ROCAL_COLOR_RGB24, 0, 1, false, area, aspect, 25,
                                                                    false, false, ROCAL_USE_USER_GIVEN_SIZE, 400, 400);
        CHECK(ctx, src);
        CHECK(ctx, rocalResize(ctx, src, 32, 32, true, ROCAL_SCALING_MODE_STRETCH));
        CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);
        CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
        std::vector<int> ids(bs), sizes(bs * 2);
        rocalGetImageId(ctx, ids.data());
        rocalGetImageSizes(ctx, sizes.data());
        std::vector<unsigned> win(bs * 4);
        unsigned seed = 0;
        CHECK(ctx, rb200_get_decoder_crop_windows(ctx, win.data(), &seed) == 0);
        fwrite(ids.data(), 4, bs, out);
        fwrite(sizes.data(), 4, bs * 2, out);
        fwrite(win.data(), 4, bs * 4, out);
        fwrite(&seed, 4, 1, out);
        RocalTensorList bl = rocalGetBoundingBoxCords(ctx);
        CHECK(ctx, bl && bl->size() == (uint64_t)bs);
        for (int i = 0; i < bs; i++) {
            CHECK(ctx, (int)bl->at(i)->dims()[0] == 1);
            float b[4];
            CHECK(ctx, bl->at(i)->copy_data(b, ROCAL_MEMCPY_HOST) == 0);
            fwrite(b, 4, 4, out);
        }
        CHECK(ctx, rocalGetStatus(ctx) == ROCAL_OK);
        rocalRelease(ctx);
    }
    fclose(out);
    printf("ok\n");
    return 0;
}
