// Emits the reference's own 4096 x 4096 ABI-smoke fixture and its scalar oracle
// (tools/cuda_backend_smoke.cu:33-49 with backend/cuda/fortai_q8_bench_spec.h),
// using the reference header from its checkout.  Run by make_golden.py only.
//   usage: fixture_from_reference ROWS WIDTH OUT_PREFIX
#include "fortai_q8_bench_spec.h"

#include <cstdio>
#include <string>

using namespace fortai_q8_bench;

static void dump(const std::string &path, const void *data, size_t bytes) {
    FILE *f = std::fopen(path.c_str(), "wb");
    std::fwrite(data, 1, bytes, f);
    std::fclose(f);
}

int main(int argc, char **argv) {
    if (argc != 4) return 2;
    const int rows = std::atoi(argv[1]);
    const int width = std::atoi(argv[2]);
    const int blocks = width / q8_block_width;
    const std::string prefix = argv[3];
    std::vector<uint8_t> weights(static_cast<size_t>(rows) * blocks * q8_block_bytes);
    std::vector<uint8_t> activation(static_cast<size_t>(blocks) * q8_block_bytes);
    std::vector<float> oracle(rows);
    fill_q8(weights, rows, blocks, 0x6f727461u, true);
    fill_q8(activation, 1, blocks, 0x6f727461u ^ 0x9e3779b9u, false);
    for (int block = 0; block < blocks; ++block) {
        activation[block * q8_block_bytes + 2] = static_cast<uint8_t>(127);
        activation[block * q8_block_bytes + 3] = static_cast<uint8_t>(-127);
    }
    make_oracle(weights, activation, rows, blocks, oracle);
    dump(prefix + ".weights.bin", weights.data(), weights.size());
    dump(prefix + ".activation.bin", activation.data(), activation.size());
    dump(prefix + ".oracle.bin", oracle.data(), oracle.size() * sizeof(float));
    return 0;
}
