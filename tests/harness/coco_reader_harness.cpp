// Prints what rb200::read_coco_annotations found, for tests/test_file_source_cpu.py:
//   harness <annotations.json> <avoid_class_remapping>
#include <cstdio>
#include <cstdlib>

#include "coco_reader.h"

int main(int argc, char** argv) {
    if (argc != 3) return 2;
    try {
        auto images = rb200::read_coco_annotations(argv[1], atoi(argv[2]) != 0);
        for (const auto& im : images) {
            printf("%s %d %d %zu", im.file_name.c_str(), im.width, im.height, im.labels.size());
            for (size_t i = 0; i < im.labels.size(); i++)
                printf(" | %d %.6f %.6f %.6f %.6f", im.labels[i], im.boxes[i * 4], im.boxes[i * 4 + 1], im.boxes[i * 4 + 2], im.boxes[i * 4 + 3]);
            printf("\n");
        }
    } catch (const std::exception& e) {
        printf("ERROR %s\n", e.what());
        return 1;
    }
    return 0;
}
