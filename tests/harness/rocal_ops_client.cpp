// A second C++ application written against include/rocal_api.h: the fixed-parameter operator calls of the reference's
// tests/cpp_api/unit_tests/unit_tests.cpp (cases 32, 34, 47-53), one graph with nine outputs, plus a detection graph
// whose boxes follow a CropMirrorNormalize. tests/test_cpp_client_gpu.py compiles it, runs it and checks every output
// against the oracle with tables rebuilt independently.
//
//   ops_client <in.bin> <out.bin>
// in.bin : int32 n, n x {int32 h, int32 w}, the n images (uint8 HWC, tightly packed),
//          int32 total_boxes, n x int32 counts, total x 4 float32 ltrb (normalized), total x int32 labels
// out.bin: per output of graph 1: int32 height, int32 width of the padded tensor, its bytes, n x 4 uint32 ROI;
//          graph 2: n x 4 uint32 crop windows, n x int32 mirror flags, then per sample int32 count, boxes, labels.
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
    if (argc != 3) return 2;
    std::vector<unsigned char> in = slurp(argv[1]);
    const unsigned char* p = in.data();
    auto rd_i32 = [&]() { int v; memcpy(&v, p, 4); p += 4; return v; };
    const int n = rd_i32();
    std::vector<int> hs(n), ws(n);
    int max_h = 0, max_w = 0;
    for (int i = 0; i < n; i++) { hs[i] = rd_i32(); ws[i] = rd_i32(); if (hs[i] > max_h) max_h = hs[i]; if (ws[i] > max_w) max_w = ws[i]; }
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
    memcpy(labels.data(), p, (size_t)total * 4);

    FILE* out = fopen(argv[2], "wb");
    if (!out) return 2;

    // ---- graph 1: the fixed-parameter operators, every one an output ----
    {
        RocalContext ctx = rocalCreate((size_t)n, ROCAL_PROCESS_GPU, 0, 1, 2, ROCAL_FP32);
        if (!ctx) return 1;
        RocalTensor src = rocalJpegExternalFileSource(ctx, ROCAL_COLOR_RGB24, false, false, false, ROCAL_USE_USER_GIVEN_SIZE,
                                                      (unsigned)max_w, (unsigned)max_h, ROCAL_DECODER_TJPEG, ROCAL_EXTSOURCE_RAW_UNCOMPRESSED);
        CHECK(ctx, src);
        RocalIntParam mirror = rocalCreateIntParameter(1);
        CHECK(ctx, rocalResizeCropMirrorFixed(ctx, src, 400, 400, true, 200, 200, mirror));
        CHECK(ctx, rocalContrastFixed(ctx, src, 30, 80, true));
        CHECK(ctx, rocalHueFixed(ctx, src, 150, true));
        CHECK(ctx, rocalSaturationFixed(ctx, src, 0.3, true));
        CHECK(ctx, rocalCropFixed(ctx, src, 224, 224, 1, true, 0, 0, 0));
        CHECK(ctx, rocalCropCenterFixed(ctx, src, 224, 224, 2, true));
        CHECK(ctx, rocalBrightnessFixed(ctx, src, 1.90, 20, true));
        CHECK(ctx, rocalColorTwistFixed(ctx, src, 0.2, 10.0, 100.0, 0.25, true));
        CHECK(ctx, rocalFlipFixed(ctx, src, 1, 0, true));
        CHECK(ctx, rocalCropFixed(ctx, src, 0, 224, 1, true, 0, 0, 0) == nullptr);        // a zero size is refused
        CHECK(ctx, rocalGetStatus(ctx) != ROCAL_OK);
        CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);
        CHECK(ctx, rocalGetAugmentationBranchCount(ctx) == 9);
        CHECK(ctx, rocalExternalSourceFeedInput(ctx, {}, false, bufs, rois, (unsigned)max_w, (unsigned)max_h, 3,
                                                ROCAL_EXTSOURCE_RAW_UNCOMPRESSED, ROCAL_NHWC, false) == ROCAL_OK);
        CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
        RocalTensorList tl = rocalGetOutputTensors(ctx);
        CHECK(ctx, tl && tl->size() == 9);
        for (int k = 0; k < 9; k++) {
            rocalTensor* t = tl->at(k);
            CHECK(ctx, t->data_type() == ROCAL_UINT8 && t->layout() == ROCAL_NHWC);
            std::vector<unsigned char> host(t->data_size());
            CHECK(ctx, t->copy_data(host.data(), ROCAL_MEMCPY_HOST) == 0);
            const int dims[2] = {(int)t->dims()[1], (int)t->dims()[2]};
            fwrite(dims, 4, 2, out);
            fwrite(host.data(), 1, host.size(), out);
            std::vector<unsigned> r4((size_t)n * 4);
            t->copy_roi(r4.data());
            fwrite(r4.data(), 4, r4.size(), out);
        }
        rocalRelease(ctx);
    }
    // ---- graph 2: boxes that follow a CropMirrorNormalize (a 160 x 120 window at anchors 0.25 / 0.75, mirrored) ----
    {
        RocalContext ctx = rocalCreate((size_t)n, ROCAL_PROCESS_GPU, 0, 1, 2, ROCAL_FP32);
        if (!ctx) return 1;
        RocalTensor src = rocalJpegExternalFileSource(ctx, ROCAL_COLOR_RGB24, false, false, false, ROCAL_USE_USER_GIVEN_SIZE,
                                                      (unsigned)max_w, (unsigned)max_h, ROCAL_DECODER_TJPEG, ROCAL_EXTSOURCE_RAW_UNCOMPRESSED);
        CHECK(ctx, src);
        std::vector<float> mean{0.f, 0.f, 0.f}, sd{1.f, 1.f, 1.f};
        RocalTensor o = rocalCropMirrorNormalize(ctx, src, 120, 160, 0.25f, 0.75f, mean, sd, true, rocalCreateIntParameter(1), ROCAL_NHWC, ROCAL_UINT8);
        CHECK(ctx, o);
        CHECK(ctx, rocalVerify(ctx) == ROCAL_OK);
        CHECK(ctx, rb200_feed_boxes(ctx, boxes.data(), labels.data(), counts.data(), (size_t)n) == 0);
        CHECK(ctx, rocalExternalSourceFeedInput(ctx, {}, false, bufs, rois, (unsigned)max_w, (unsigned)max_h, 3,
                                                ROCAL_EXTSOURCE_RAW_UNCOMPRESSED, ROCAL_NHWC, false) == ROCAL_OK);
        CHECK(ctx, rocalRun(ctx) == ROCAL_OK);
        std::vector<unsigned> win((size_t)n * 4);
        CHECK(ctx, rb200_get_crop_windows(ctx, o, win.data()) == 0);
        fwrite(win.data(), 4, win.size(), out);
        RocalTensorList bl = rocalGetBoundingBoxCords(ctx), ll = rocalGetBoundingBoxLabel(ctx);
        CHECK(ctx, bl && ll && bl->size() == (uint64_t)n && ll->size() == (uint64_t)n);
        for (int i = 0; i < n; i++) {
            int cnt = (int)bl->at(i)->dims()[0];
            fwrite(&cnt, 4, 1, out);
            std::vector<float> b((size_t)cnt * 4);
            std::vector<int> l(cnt);
            CHECK(ctx, bl->at(i)->copy_data(b.data(), ROCAL_MEMCPY_HOST) == 0 && ll->at(i)->copy_data(l.data(), ROCAL_MEMCPY_HOST) == 0);
            fwrite(b.data(), 4, b.size(), out);
            fwrite(l.data(), 4, l.size(), out);
        }
        CHECK(ctx, rocalGetStatus(ctx) == ROCAL_OK);
        rocalRelease(ctx);
    }
    fclose(out);
    printf("ok\n");
    return 0;
}
