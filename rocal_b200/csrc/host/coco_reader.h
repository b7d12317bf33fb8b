// COCO annotation reader behind rocalCreateCOCOReader / rocalJpegCOCOFileSource.
//
// What it takes from the annotation file follows the reference's reader
// (rocAL/source/meta_data/coco_meta_data_reader.cpp:140-325):
//   images[]      id, file_name, width, height
//   categories[]  id; classes are renumbered 1, 2, ... in order of appearance unless class remapping is avoided
//   annotations[] image_id, category_id, bbox = [x, y, w, h] in pixels -> ltrb = (x, y, x + w, y + h); crowd
//                 annotations are kept, as the reference keeps them for the bounding-box metadata type
// Everything else in the file is skipped. The reference stores pixel coordinates and rescales them along the
// graph; this pipeline's metadata space is normalized ltrb (as rb200_feed_boxes takes it), so boxes are divided by
// the image's width and height from the file.
#pragma once
#include <map>
#include <string>
#include <vector>

namespace rb200 {

struct CocoImage {
    std::string file_name;
    long id = 0;                 // "id" of the images entry (what rocalGetImageId reports)
    int width = 0, height = 0;
    std::vector<float> boxes;    // normalized ltrb, 4 per annotation, in file order
    std::vector<int> labels;
};

// Parses the file; throws std::runtime_error on unreadable or malformed input. The result is ordered by file name.
std::vector<CocoImage> read_coco_annotations(const std::string& json_path, bool avoid_class_remapping);

}  // namespace rb200
