// CPU restatement of the fused-network forward path and training step in plain C++ (TEST INFRASTRUCTURE, not product code).
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
// The training step (oracle_network_train_step) follows the backward math of tests_cpp/test_against_eigen2.cpp:169-206
// (delta = Act'(pre) * adj, adjBias = row sums of delta, adjW = delta * in^T, adjIn = W^T * delta), the grid adjoint of
// kernels/encoding_hashgrid.cuh:130-140 (one atomic float add per corner and feature), and the loss and optimiser the
// reference's users write around it (tests_py/qmlp_tests/test_network_image.py:43,51-53: mse loss, torch Adam).
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

// ---- training step ---------------------------------------------------------------------------------------------------
namespace {

inline float activate_adjoint(int a, float x, float g)
{
    switch (a) {
    case 0: return x > 0.f ? g : 0.f;
    case 1: return x > 0.f ? g : g * std::exp(x);
    case 2: return std::cos(x) * g;
    default: return g;
    }
}

// kernels/encoding_hashgrid.cuh:345-422 (parameter part): grad[row + i] += w_corner * adj[i], atomically
void grid_adjoint_point(const OracleEncoding& e, const float* x, const float* adj, float* grad)
{
    const int D = e.n_in, F = e.n_features;
    float pos[6];
    for (int i = 0; i < D; ++i) pos[i] = (x[e.start_in + i] - e.box_min[i]) * e.box_inv_size[i];
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
        const float* af = adj + (e.concat ? l * F : 0);
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
            float* row = grad + lv.memory_offset + static_cast<int64_t>(idx) * F;
            for (int i = 0; i < F; ++i) {
                const float v = w * af[i];
#pragma omp atomic
                row[i] += v;
            }
        }
    }
}

// torch.optim.Adam without amsgrad or weight decay; step is 1-based; the gradient is cleared for the next step
void adam_update(float* p, float* g, float* m, float* v, int64_t count, int step, float lr, float beta1, float beta2, float eps)
{
    const double bc1 = 1.0 - std::pow(static_cast<double>(beta1), step);
    const double bc2 = 1.0 - std::pow(static_cast<double>(beta2), step);
    const float stepSize = static_cast<float>(lr / bc1);
    const float invSqrtBc2 = static_cast<float>(1.0 / std::sqrt(bc2));
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const float gi = g[i];
        const float mi = beta1 * m[i] + (1.f - beta1) * gi;
        const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        p[i] -= stepSize * mi / (std::sqrt(vi) * invSqrtBc2 + eps);
        g[i] = 0.f;
    }
}

} // namespace

extern "C" {

// One training step on the host: forward with the pre-activations kept, L2-loss gradient
// 2 (out - target) / (n_global * num_outputs), backward through the layers, weight / bias / table gradients, Adam.
// The network's parameter vector and every grid table are updated in place (they are the arrays net points to);
// grad_*, m_*, v_* have the same lengths (grad must be zero on entry and is zero again on return). `update` = 0 stops
// after the gradients (they are then left in grad_* for a comparison). Returns the sum of squared errors.
double oracle_network_train_step(const OracleNetwork* net, const float* x, const float* target, int64_t n, int64_t n_global,
                                 float* grad_params, float* m_params, float* v_params, int64_t num_params,
                                 float* const* grad_tables, float* const* m_tables, float* const* v_tables,
                                 const int64_t* table_counts, int step, float lr, float beta1, float beta2, float eps,
                                 int update, int num_threads)
{
    constexpr int BLOCK = 64;
    const int NL = net->num_layers;
    int maxw = 0, sumOut = 0;
    for (int l = 0; l < NL; ++l) {
        if (net->layers[l].channels_in > maxw) maxw = net->layers[l].channels_in;
        if (net->layers[l].channels_out > maxw) maxw = net->layers[l].channels_out;
        sumOut += net->layers[l].channels_out;
    }
    const int cin0 = net->layers[0].channels_in;
    const int64_t blocks = (n + BLOCK - 1) / BLOCK;
    const float lossScale = static_cast<float>(2.0 / (static_cast<double>(n_global > 0 ? n_global : n) * net->num_outputs));
    double lossSum = 0.0;
#ifdef _OPENMP
    if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
#pragma omp parallel reduction(+ : lossSum)
    {
        // per thread: layer inputs and pre-activations of one block, two adjoint buffers, a private copy of the
        // (small) network gradient
        std::vector<float> ins(static_cast<size_t>(BLOCK) * (cin0 + sumOut)), pres(static_cast<size_t>(BLOCK) * sumOut);
        std::vector<float> adjA(static_cast<size_t>(BLOCK) * maxw), adjB(static_cast<size_t>(BLOCK) * maxw);
        std::vector<float> gp(static_cast<size_t>(num_params), 0.f);
#pragma omp for schedule(static)
        for (int64_t blk = 0; blk < blocks; ++blk) {
            const int64_t p0 = blk * BLOCK;
            const int m = static_cast<int>(n - p0 < BLOCK ? n - p0 : BLOCK);
            // encodings
            float* in0 = ins.data();
            for (int r = 0; r < m; ++r) {
                float* row = in0 + static_cast<size_t>(r) * cin0;
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
            // forward, keeping the input and the pre-activation of every layer
            float* in = in0;
            float* pre = pres.data();
            for (int l = 0; l < NL; ++l) {
                const OracleLayer& L = net->layers[l];
                const float* W = net->params + L.weights_start;
                const float* B = L.use_bias ? net->params + L.bias_start : nullptr;
                float* out = in + static_cast<size_t>(BLOCK) * L.channels_in;
                for (int r = 0; r < m; ++r) {
                    const float* a = in + static_cast<size_t>(r) * L.channels_in;
                    for (int c = 0; c < L.channels_out; ++c) {
                        const float* w = W + static_cast<size_t>(c) * L.channels_in;
                        float s = 0.f;
#pragma omp simd reduction(+ : s)
                        for (int k = 0; k < L.channels_in; ++k) s += w[k] * a[k];
                        if (B) s += B[c];
                        pre[static_cast<size_t>(r) * L.channels_out + c] = s;
                        out[static_cast<size_t>(r) * L.channels_out + c] = activate(L.activation, s);
                    }
                }
                in = out;
                pre += static_cast<size_t>(BLOCK) * L.channels_out;
            }
            // loss gradient on the first num_outputs channels of the last layer's output
            const OracleLayer& LL = net->layers[NL - 1];
            float* adj = adjA.data();
            float* nxt = adjB.data();
            for (int r = 0; r < m; ++r)
                for (int c = 0; c < LL.channels_out; ++c) {
                    float g = 0.f;
                    if (c < net->num_outputs) {
                        const float d = in[static_cast<size_t>(r) * LL.channels_out + c] - target[(p0 + r) * net->num_outputs + c];
                        lossSum += static_cast<double>(d) * d;
                        g = lossScale * d;
                    }
                    adj[static_cast<size_t>(r) * LL.channels_out + c] = g;
                }
            // backward
            for (int l = NL - 1; l >= 0; --l) {
                const OracleLayer& L = net->layers[l];
                pre -= static_cast<size_t>(BLOCK) * L.channels_out;
                in -= static_cast<size_t>(BLOCK) * L.channels_in;     // input of layer l
                const float* W = net->params + L.weights_start;
                float* gW = gp.data() + L.weights_start;
                float* gB = L.use_bias ? gp.data() + L.bias_start : nullptr;
                for (int r = 0; r < m; ++r) {
                    float* d = adj + static_cast<size_t>(r) * L.channels_out;
                    const float* pr = pre + static_cast<size_t>(r) * L.channels_out;
                    const float* a = in + static_cast<size_t>(r) * L.channels_in;
                    float* ai = nxt + static_cast<size_t>(r) * L.channels_in;
                    for (int k = 0; k < L.channels_in; ++k) ai[k] = 0.f;
                    for (int c = 0; c < L.channels_out; ++c) {
                        const float dc = activate_adjoint(L.activation, pr[c], d[c]);
                        if (dc == 0.f) continue;
                        if (gB) gB[c] += dc;
                        float* gw = gW + static_cast<size_t>(c) * L.channels_in;
                        const float* w = W + static_cast<size_t>(c) * L.channels_in;
#pragma omp simd
                        for (int k = 0; k < L.channels_in; ++k) {
                            gw[k] += dc * a[k];
                            ai[k] += dc * w[k];
                        }
                    }
                }
                float* t = adj; adj = nxt; nxt = t;
            }
            // encoding adjoints (parameter gradients only: the training step asks for no input gradient)
            for (int r = 0; r < m; ++r) {
                const float* xr = x + (p0 + r) * net->num_inputs;
                const float* a = adj + static_cast<size_t>(r) * cin0;
                int off = 0;
                for (int e = 0; e < net->num_encodings; ++e) {
                    const OracleEncoding& enc = net->encodings[e];
                    if (enc.is_grid && grad_tables && grad_tables[e]) grid_adjoint_point(enc, xr, a + off, grad_tables[e]);
                    off += enc.num_outputs;
                }
            }
        }
#pragma omp critical
        for (int64_t i = 0; i < num_params; ++i) grad_params[i] += gp[static_cast<size_t>(i)];
    }
    if (update) {
        adam_update(const_cast<float*>(net->params), grad_params, m_params, v_params, num_params, step, lr, beta1, beta2, eps);
        for (int e = 0; e < net->num_encodings; ++e)
            if (net->encodings[e].is_grid && grad_tables && grad_tables[e])
                adam_update(const_cast<float*>(net->encodings[e].table), grad_tables[e], m_tables[e], v_tables[e], table_counts[e],
                            step, lr, beta1, beta2, eps);
    }
    return lossSum;
}

} // extern "C"
