// Prints what the reference's own safetensors loader (src/model/safetensors_loader.cpp) finds in a
// file: for every tensor its dtype code, shape, byte size and a 64-bit FNV-1a hash of its bytes, as
// one JSON object on standard output.  Built against the reference's sources by
// make_safetensors_golden.py (with nvcc, because the reference's tensor class includes the CUDA
// runtime; nothing here calls it).
#include "model/safetensors_loader.h"

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

int main(int argc, char** argv) {
    if (argc != 2) {
        std::fprintf(stderr, "usage: dump_reference_safetensors FILE\n");
        return 2;
    }
    mini_infer::SafetensorsLoader loader(argv[1]);
    std::vector<std::string> names;
    for (const auto& kv : loader.tensors()) names.push_back(kv.first);
    std::sort(names.begin(), names.end());
    std::printf("{");
    for (size_t i = 0; i < names.size(); ++i) {
        const mini_infer::WeightInfo* w = loader.find(names[i]);
        uint64_t h = 1469598103934665603ull;
        const uint8_t* p = loader.data_section() + w->byte_offset;
        for (size_t b = 0; b < w->byte_size; ++b) { h ^= p[b]; h *= 1099511628211ull; }
        std::printf("%s\"%s\": {\"dtype\": %d, \"shape\": [", i ? ", " : "", names[i].c_str(), (int)w->dtype);
        for (size_t d = 0; d < w->shape.size(); ++d) std::printf("%s%lld", d ? ", " : "", (long long)w->shape[d]);
        std::printf("], \"nbytes\": %zu, \"fnv64\": \"%016llx\"}", w->byte_size, (unsigned long long)h);
    }
    std::printf("}\n");
    return 0;
}
