// Prints the batch sequence of rb200::FileSource for tests/test_file_source_cpu.py:
//   harness <root> <batch> <shard_id> <shard_count> <shuffle> <loop_batches> <policy> <pad_repeat> [file_list]
#include <cstdio>
#include <cstdlib>

#include "file_source.h"

using namespace rb200;

int main(int argc, char** argv) {
    if (argc != 9 && argc != 10) return 2;
    try {
        const int loop_batches = atoi(argv[6]);
        FileSource fs = argc == 10
                            ? FileSource(read_file_list(argv[9], argv[1]), false, (size_t)atoi(argv[2]), (unsigned)atoi(argv[3]),
                                         (unsigned)atoi(argv[4]), atoi(argv[5]) != 0, loop_batches > 0, atoi(argv[7]), atoi(argv[8]) != 0, 7)
                            : FileSource(argv[1], (size_t)atoi(argv[2]), (unsigned)atoi(argv[3]), (unsigned)atoi(argv[4]),
                                         atoi(argv[5]) != 0, loop_batches > 0, atoi(argv[7]), atoi(argv[8]) != 0, 7);
        printf("N=%zu shard=%zu per=%zu\n", fs.dataset_size(), fs.shard_size(), fs.batches_per_epoch());
        FileBatch b;
        int k = 0;
        while (fs.next(b)) {
            for (size_t i = 0; i < b.names.size(); i++) printf("%s:%d ", b.names[i].c_str(), b.labels[i]);
            printf("| pad %zu\n", b.padded);
            if (loop_batches > 0 && ++k >= loop_batches) break;
        }
    } catch (const std::exception& e) {
        printf("ERROR %s\n", e.what());
        return 1;
    }
    return 0;
}
