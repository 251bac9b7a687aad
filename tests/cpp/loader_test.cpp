// Exercises the C++ loader mirror (rusty_b200/host/rusty_loader.hpp).
//   loader_test info <file>                       names, dtypes, shapes (host only: runs without a GPU)
//   loader_test shard <file> <name> <rank> <world>  FNV-1a checksums of the rank's weight bytes / scales / biases (host only);
//                                                  shard_kn: the same with the matrix read as [in,out] (column shards)
//   loader_test gpu <file> <name>                  upload both ways on device 0 and compare dequantise-then-matmul
//                                                  with the fused linear (needs a GPU); prints "ok"
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>

#include "rusty_loader.hpp"

using namespace rusty;

static unsigned long long fnv(const void* p, size_t n) {
    const unsigned char* b = static_cast<const unsigned char*>(p);
    unsigned long long h = 1469598103934665603ull;
    for (size_t i = 0; i < n; ++i) h = (h ^ b[i]) * 1099511628211ull;
    return h;
}

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const std::string mode = argv[1];
    try {
        WeightsContext w;
        w.load_file(argv[2]);
        if (mode == "info") {
            for (int i = 3; i < argc; ++i) {
                const TensorInfo* t = w.get_tensor_info(argv[i]);
                if (!t) {
                    std::printf("%s missing\n", argv[i]);
                    continue;
                }
                std::printf("%s %s", argv[i], t->dtype.c_str());
                for (size_t d : t->shape) std::printf(" %zu", d);
                std::printf(" quantized=%d\n", (int)w.is_quantized(std::string(argv[i]).substr(0, std::string(argv[i]).rfind('.'))));
            }
            return 0;
        }
        if ((mode == "shard" || mode == "shard_kn") && argc == 6) {
            const auto s = w.quantized_shard(argv[3], mode == "shard" ? RUSTY_CUDA_LAYOUT_NK : RUSTY_CUDA_LAYOUT_KN, std::atoi(argv[4]), std::atoi(argv[5]));
            std::printf("%zu %zu %zu %llu %llu %llu\n", s.rows, s.cols, s.groups, fnv(s.q, s.rows * s.cols), fnv(s.scales, s.groups * 4),
                        fnv(s.biases, s.groups * 4));
            return 0;
        }
        if (mode == "gpu" && argc == 4) {
            CudaContext ctx(0);
            ComputeEngine engine(ctx);
            const std::string name = argv[3];
            UnifiedTensor wf = w.upload_quantized(name, ctx, engine);  // [N, K] f32, the reference's load path
            const size_t N = wf.shape[0], K = wf.shape[1], M = 6;
            std::mt19937 rng(3);
            std::normal_distribution<float> nd(0.f, 1.f);
            std::vector<float> x(M * K);
            for (auto& e : x) e = nd(rng);
            auto tx = UnifiedTensor::make(ctx, x.data(), {M, K});
            auto ref = UnifiedTensor::empty(ctx, {M, N});
            engine.matmul_bt(ctx, tx, wf, ref);  // x . W^T over the dequantised copy
            Linear lin = Linear::from_quantized(ctx, w.upload_qlinear(name, ctx, RUSTY_CUDA_LAYOUT_NK));
            auto got = lin.forward(engine, tx).to_vec(ctx);
            auto want = ref.to_vec(ctx);
            double mref = 0, merr = 0;
            for (size_t i = 0; i < want.size(); ++i) {
                mref = std::fmax(mref, std::fabs(want[i]));
                merr = std::fmax(merr, std::fabs((double)want[i] - got[i]));
            }
            if (!(mref > 0 && merr / mref <= 1e-5)) {
                std::fprintf(stderr, "mismatch %g / %g\n", merr, mref);
                return 1;
            }
            std::printf("ok\n");
            return 0;
        }
    } catch (const LoaderError& e) {
        std::printf("LoaderError %s\n", e.kind.c_str());
        return 3;
    }
    return 2;
}
