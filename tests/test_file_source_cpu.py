"""The folder reader behind rocalJpegFileSource (rocal_b200/csrc/host/file_source.cpp), compiled into a small
harness: class numbering, extension filter, shard ranges, last-batch policies, seeded shuffle, looping. The harnesses
are built with the address and undefined-behaviour sanitizers: a finding aborts the run and fails the test."""
import os
import subprocess

import pytest

SANITIZE = ["-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer"]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "rocal_b200", "csrc", "host")


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    d = tmp_path_factory.mktemp("fs")
    exe = str(d / "harness")
    subprocess.run(["g++", "-std=c++17", "-O1"] + SANITIZE + ["-I", HOST, os.path.join(ROOT, "tests", "harness", "file_source_harness.cpp"),
                    os.path.join(HOST, "file_source.cpp"), "-o", exe], check=True)
    data = d / "data"
    for cls, count in (("cat", 3), ("dog", 4), ("emu", 2)):
        (data / cls).mkdir(parents=True)
        for i in range(count):
            (data / cls / ("%s%d.jpg" % (cls, i))).write_bytes(b"x")
    (data / "cat" / "readme.txt").write_text("not an image")
    (data / "dog" / "DOG9.JPEG").write_bytes(b"x")          # upper-case extension counts; sorts before the lower-case names
    flat = d / "flat"
    flat.mkdir()
    for i in range(3):
        (flat / ("f%d.jpeg" % i)).write_bytes(b"x")

    def run(root, batch, shard_id, shard_count, shuffle=0, loop_batches=0, policy=0, pad_repeat=0, file_list=None):
        r = subprocess.run([exe, str(root), str(batch), str(shard_id), str(shard_count), str(shuffle), str(loop_batches),
                            str(policy), str(pad_repeat)] + ([str(file_list)] if file_list else []),
                           capture_output=True, text=True)
        assert "Sanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-2000:]
        out = r.stdout.strip().splitlines()
        if out and out[0].startswith("ERROR"):
            return out[0], [], []
        return out[0], [ln.split("|")[0].split() for ln in out[1:]], [int(ln.split("pad")[1]) for ln in out[1:]]
    return run, data, flat, d


def test_classes_order_and_fill(harness):
    run, data, flat, _ = harness
    head, batches, pads = run(data, 4, 0, 1)
    assert head == "N=10 shard=10 per=3"
    flat_list = [x for b in batches for x in b]
    assert flat_list[:10] == ["cat0.jpg:0", "cat1.jpg:0", "cat2.jpg:0", "DOG9.JPEG:1", "dog0.jpg:1", "dog1.jpg:1", "dog2.jpg:1",
                              "dog3.jpg:1", "emu0.jpg:2", "emu1.jpg:2"]
    assert flat_list[10:] == ["cat0.jpg:0", "cat1.jpg:0"] and pads == [0, 0, 2]       # FILL wraps to the shard's start
    _, batches, pads = run(data, 4, 0, 1, pad_repeat=1)
    assert batches[-1][2:] == ["emu1.jpg:2", "emu1.jpg:2"] and pads[-1] == 2            # ... or repeats the last sample
    head, batches, _ = run(flat, 2, 0, 1)
    assert head == "N=3 shard=3 per=2" and all(x.endswith(":0") for b in batches for x in b)


def test_shards_and_drop(harness):
    run, data, _, _ = harness
    seen = []
    for shard in range(3):
        head, batches, pads = run(data, 2, shard, 3, policy=1)
        n = int(head.split("shard=")[1].split()[0])
        assert n == 10 * (shard + 1) // 3 - 10 * shard // 3
        assert len(batches) == n // 2 and all(p == 0 for p in pads)                     # DROP: whole batches only
        seen += [x for b in batches for x in b]
    assert len(set(seen)) == len(seen)                                                   # shards do not overlap
    assert run(data, 2, 3, 3)[0].startswith("ERROR")


def test_shuffle_and_loop(harness):
    run, data, _, _ = harness
    _, a, _ = run(data, 5, 0, 1, shuffle=1)
    _, b, _ = run(data, 5, 0, 1, shuffle=1)
    assert a == b                                                                        # seeded
    assert sorted(x for bt in a for x in bt) == sorted(x for bt in run(data, 5, 0, 1)[1] for x in bt)
    assert [x for bt in a for x in bt] != [x for bt in run(data, 5, 0, 1)[1] for x in bt]
    _, looped, _ = run(data, 5, 0, 1, shuffle=1, loop_batches=4)
    assert len(looped) == 4 and looped[:2] == a and looped[2:] != a                      # the next epoch is reshuffled


def test_coco_annotation_reader(tmp_path):
    """The COCO reader: categories renumbered in file order (or kept), bbox xywh -> normalized ltrb, annotations that
    precede the images section, escaped strings, nested values it has to skip, crowd annotations kept, images without
    annotations kept, unknown images dropped, output sorted by file name."""
    import json
    exe = str(tmp_path / "coco")
    subprocess.run(["g++", "-std=c++17", "-O1"] + SANITIZE + ["-I", HOST, os.path.join(ROOT, "tests", "harness", "coco_reader_harness.cpp"),
                    os.path.join(HOST, "coco_reader.cpp"), "-o", exe], check=True)
    doc = {
        "info": {"description": "synthetic \"set\"", "nested": [1, [2, {"a": None}], True], "year": 2026},
        "annotations": [
            {"id": 1, "image_id": 20, "category_id": 18, "bbox": [10.0, 20.0, 30.0, 40.0], "iscrowd": 0, "segmentation": [[1, 2, 3, 4]]},
            {"id": 2, "image_id": 10, "category_id": 3, "bbox": [0, 0, 50, 25], "iscrowd": 1, "area": 1250.5},
            {"id": 3, "image_id": 20, "category_id": 3, "bbox": [5.5, 6.5, 7.0, 8.0], "iscrowd": 0},
            {"id": 4, "image_id": 99, "category_id": 3, "bbox": [1, 1, 1, 1]},
        ],
        "categories": [{"id": 3, "name": "car", "supercategory": "vehicle"}, {"id": 18, "name": "dog"}],
        "images": [
            {"id": 20, "file_name": "b_img.jpg", "width": 200, "height": 100, "license": 1},
            {"id": 10, "file_name": "a_img.jpg", "height": 50, "width": 100},
            {"id": 30, "file_name": "c_empty.jpg", "width": 64, "height": 64},
        ],
    }
    path = tmp_path / "ann.json"
    path.write_text(json.dumps(doc, indent=1))

    def run(avoid):
        r = subprocess.run([exe, str(path), str(avoid)], capture_output=True, text=True)
        assert "Sanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-2000:]
        return [ln.split(" | ") for ln in r.stdout.strip().splitlines()]

    rows = run(0)
    assert [r[0] for r in rows] == ["a_img.jpg 100 50 1", "b_img.jpg 200 100 2", "c_empty.jpg 64 64 0"]
    assert rows[0][1] == "1 0.000000 0.000000 0.500000 0.500000"                 # category 3 -> class 1
    assert rows[1][1] == "2 0.050000 0.200000 0.200000 0.600000"                 # category 18 -> class 2
    assert rows[1][2] == "1 0.027500 0.065000 0.062500 0.145000"
    rows = run(1)
    assert rows[0][1].startswith("3 ") and rows[1][1].startswith("18 ")
    bad = tmp_path / "bad.json"
    bad.write_text('{"images": [ {"id": 1, "file_name": "x.jpg" ')
    assert subprocess.run([exe, str(bad), "0"], capture_output=True, text=True).stdout.startswith("ERROR")


def test_file_list(harness):
    """A "file_name label" list (rocalCreateLabelReader with file_list_path): list order and list labels, names relative
    to the root, the reported name without its folder, unparsable lines and non-JPEG names skipped."""
    run, data, _, d = harness
    lst = d / "list.txt"
    lst.write_text("dog/dog2.jpg 7\nemu/emu0.jpg 3\n# a comment\ncat/readme.txt 1\ncat/cat1.jpg 0\nbroken_line\ndog/DOG9.JPEG 7\n")
    head, batches, pads = run(data, 2, 0, 1, file_list=lst)
    assert head == "N=4 shard=4 per=2"
    assert [x for b in batches for x in b] == ["dog2.jpg:7", "emu0.jpg:3", "cat1.jpg:0", "DOG9.JPEG:7"] and pads == [0, 0]
    head, _, _ = run(data, 2, 0, 1, file_list=d / "missing.txt")
    assert head.startswith("ERROR")
