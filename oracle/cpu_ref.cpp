// CPU restatement of the fused-network forward path in plain C++ (TEST INFRASTRUCTURE, not product code).
//
// It exists to time the reference algorithm on host cores (the CPU-baseline leg of the benchmark) and to cross-check
// the numpy oracle. Only tests/, the smoke check and the benchmark's CPU-baseline / reference arm may build or call it;
// the product path never does.
//
// The reference's own CPU path is the float Eigen::MatrixX forward written inside its tests
// (tests_cpp/test_against_eigen2.cpp:134-149: out = Act(W * in + b) per layer, activations as
// tests_cpp/test_against_eigen.h:33-87). Eigen is not available here (a FetchContent download,
// tests_cpp/Eigen/CMakeLists.txt:1-15), so the same float math is written out: one row-blocked GEMM per layer,
// OpenMP over blocks of points. The grid encoder follows src_cpp/include/qmlp/kernels/encoding_hashgrid.cuh:18-60
// (index), :174-215 (N-linear weights), :267-336 (forward); identity follows kernels/encoding_identity.cuh:16-25.
// Parity status: pinned only through the numpy oracle (tests/test_oracle.py compares both); see that module's header.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

struct OracleLevel {
    int64_t memory_offset;
    int32_t resolution;
    int32_t hash_grid_size;
    int32_t hashed;
    int32_t pad;
};

struct OracleEncoding {
    int32_t is_grid;      // 0: identity, 1: grid
    int32_t start_in, n_in;
    int32_t num_outputs;
    int32_t n_levels, n_features;
    int32_t concat;
    int32_t pad;
    float box_min[6], box_inv_size[6];
    const OracleLevel* levels;
    const float* table;
};

struct OracleLayer {
    int32_t channels_in, channels_out; // padded
    int32_t use_bias;
    int32_t activation;                // 0 relu, 1 celu, 2 sine, 3 identity
    int64_t weights_start, bias_start;
};

struct OracleNetwork {
    int32_t num_inputs, num_outputs;
    int32_t num_encodings, num_layers;
    const OracleEncoding* encodings;
    const OracleLayer* layers;
    const float* params; // flat parameter vector, already converted to float
};

} // extern "C"

namespace {

const uint32_t PRIMES[6] = {1u, 43857811u, 83857661u, 73856093u, 19349663u, 834927u};

inline float activate(int a, float x)
{
    switch (a) {
    case 0: return x > 0.f ? x : 0.f;
    case 1: return x > 0.f ? x : std::exp(x) - 1.f;
    case 2: return std::sin(x);
    default: return x;
    }
}

void grid_forward_point(const OracleEncoding& e, const float* x, float* out)
{
    const int D = e.n_in, F = e.n_features;
    float pos[6];
    for (int i = 0; i < D; ++i) pos[i] = (x[e.start_in + i] - e.box_min[i]) * e.box_inv_size[i];
    if (!e.concat) for (int i = 0; i < F; ++i) out[i] = 0.f;
    for (int l = 0; l < e.n_levels; ++l) {
        const OracleLevel& lv = e.levels[l];
        uint32_t lo[6], hi[6];
        float f[6];
        const int rm1 = lv.resolution - 1;
        for (int i = 0; i < D; ++i) {
            const float p = pos[i] * static_cast<float>(rm1);
            const int ip = static_cast<int>(p);
            const int a = ip < 0 ? 0 : (ip > rm1 ? rm1 : ip);
            const int b = ip + 1 < 0 ? 0 : (ip + 1 > rm1 ? rm1 : ip + 1);
            lo[i] = static_cast<uint32_t>(a);
            hi[i] = static_cast<uint32_t>(b);
            f[i] = p - static_cast<float>(a);
        }
        float feat[16];
        for (int i = 0; i < F; ++i) feat[i] = 0.f;
        for (int c = 0; c < (1 << D); ++c) {
            uint32_t idx;
            if (lv.hashed) {
                idx = ((c & 1) ? hi[0] : lo[0]) * PRIMES[0];
                for (int k = 1; k < D; ++k) idx = ((((c >> k) & 1) ? hi[k] : lo[k]) * PRIMES[k]) ^ idx;
                idx = idx % static_cast<uint32_t>(lv.hash_grid_size);
            } else {
                idx = (c & 1) ? hi[0] : lo[0];
                for (int k = 1; k < D; ++k) idx = (((c >> k) & 1) ? hi[k] : lo[k]) + idx * static_cast<uint32_t>(lv.resolution);
            }
            float w = 1.f;
            for (int k = D - 1; k >= 0; --k) w *= ((c >> k) & 1) ? f[k] : (1.f - f[k]);
            const float* row = e.table + lv.memory_offset + static_cast<int64_t>(idx) * F;
            for (int i = 0; i < F; ++i) feat[i] += w * row[i];
        }
        if (e.concat) for (int i = 0; i < F; ++i) out[l * F + i] = feat[i];
        else for (int i = 0; i < F; ++i) out[i] += feat[i];
    }
}

} // namespace

extern "C" {

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// x: (n, num_inputs) row-major float; out: (n, num_outputs) row-major float.
// num_threads <= 0: all available.
void oracle_network_forward(const OracleNetwork* net, const float* x, int64_t n, float* out, int num_threads)
{
    constexpr int BLOCK = 64;
    int maxw = 0;
    for (int l = 0; l < net->num_layers; ++l) {
        if (net->layers[l].channels_in > maxw) maxw = net->layers[l].channels_in;
        if (net->layers[l].channels_out > maxw) maxw = net->layers[l].channels_out;
    }
    const int64_t blocks = (n + BLOCK - 1) / BLOCK;
#ifdef _OPENMP
    if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
#pragma omp parallel
    {
        std::vector<float> a(static_cast<size_t>(BLOCK) * maxw), b(static_cast<size_t>(BLOCK) * maxw);
#pragma omp for schedule(static)
        for (int64_t blk = 0; blk < blocks; ++blk) {
            const int64_t p0 = blk * BLOCK;
            const int m = static_cast<int>(n - p0 < BLOCK ? n - p0 : BLOCK);
            float* cur = a.data();
            float* nxt = b.data();
            const int cin0 = net->layers[0].channels_in;
            // encodings -> (m, cin0), padding channels zero
            for (int r = 0; r < m; ++r) {
                float* row = cur + static_cast<size_t>(r) * cin0;
                std::memset(row, 0, sizeof(float) * cin0);
                int off = 0;
                const float* xr = x + (p0 + r) * net->num_inputs;
                for (int e = 0; e < net->num_encodings; ++e) {
                    const OracleEncoding& enc = net->encodings[e];
                    if (enc.is_grid) grid_forward_point(enc, xr, row + off);
                    else for (int i = 0; i < enc.n_in; ++i) row[off + i] = xr[enc.start_in + i];
                    off += enc.num_outputs;
                }
            }
            // layers: out = Act(in * W^T + b)
            for (int l = 0; l < net->num_layers; ++l) {
                const OracleLayer& L = net->layers[l];
                const float* W = net->params + L.weights_start;
                const float* B = L.use_bias ? net->params + L.bias_start : nullptr;
                for (int r = 0; r < m; ++r) {
                    const float* in = cur + static_cast<size_t>(r) * L.channels_in;
                    float* o = nxt + static_cast<size_t>(r) * L.channels_out;
                    for (int c = 0; c < L.channels_out; ++c) {
                        const float* w = W + static_cast<size_t>(c) * L.channels_in;
                        float s = 0.f;
#pragma omp simd reduction(+ : s)
                        for (int k = 0; k < L.channels_in; ++k) s += w[k] * in[k];
                        if (B) s += B[c];
                        o[c] = activate(L.activation, s);
                    }
                }
                float* t = cur; cur = nxt; nxt = t;
            }
            const int cl = net->layers[net->num_layers - 1].channels_out;
            for (int r = 0; r < m; ++r)
                for (int c = 0; c < net->num_outputs; ++c) out[(p0 + r) * net->num_outputs + c] = cur[static_cast<size_t>(r) * cl + c];
        }
    }
}

} // extern "C"
