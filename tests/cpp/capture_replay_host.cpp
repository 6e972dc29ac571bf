// Native host of the flat C ABI, with no Python and no torch in the process: what a Rust caller of
// include/baracuda_kernels_q.h does, written against the CUDA runtime only.  It follows the pattern of the reference's
// graph test (crates/baracuda-kernels/tests/capture_replay_gather_gemv.rs:1-24): a ZEROED output, an eager warm launch,
// then the same call captured into a CUDA graph and replayed WITHOUT re-zeroing, so a replay that drops or mis-writes
// an element diverges from the host-computed expectation.  On top of that the inputs are rewritten between replays:
// a replay must read the buffers' current contents.  Covered: the decode GEMV (both weight layouts), the one-launch
// decode step from bf16 activations, the W8A8 GEMM whose tensor maps travel as kernel parameters, and the C++ Plan layer
// (QuantizedLinearPlan as a chain of dependent launches inside one graph, SmoothQuantLinearPlan).
//
// Build: g++ -std=c++17 -O1 -I include -I <cuda>/include capture_replay_host.cpp -L baracuda_b200
//        -lbaracuda_kernels_q -L <cuda>/lib64 -lcudart ; prints "capture_replay_host ok".

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "baracuda_kernels_q.h"
#include "baracuda_kernels_q_plan.hpp"

#define CK(x)                                                                                  \
    do {                                                                                       \
        cudaError_t e_ = (x);                                                                  \
        if (e_ != cudaSuccess) {                                                               \
            std::printf("%s:%d cuda error %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return 1;                                                                          \
        }                                                                                      \
    } while (0)
#define REQUIRE(c)                                                     \
    do {                                                               \
        if (!(c)) {                                                    \
            std::printf("%s:%d failed: %s\n", __FILE__, __LINE__, #c); \
            return 1;                                                  \
        }                                                              \
    } while (0)

namespace {

uint32_t lcg(uint32_t& s) {
    s = s * 1664525u + 1013904223u;
    return s >> 8;
}

// f32 -> bf16, round to nearest even (the oracle's codec: crates/baracuda-kernelgen/src/oracle.rs:397-404)
uint16_t bf16_rne(float x) {
    uint32_t b;
    std::memcpy(&b, &x, 4);
    if ((b & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((b >> 16) | 0x40);
    b += 0x7fffu + ((b >> 16) & 1u);
    return static_cast<uint16_t>(b >> 16);
}

float bf16_to_f32(uint16_t h) {
    uint32_t b = static_cast<uint32_t>(h) << 16;
    float x;
    std::memcpy(&x, &b, 4);
    return x;
}

// out[r, j] = bf16((sa[r] * sb[j]) * (float)sum_k a[r,k] * w(j,k)) -- baracuda_quantize_compose.cuh:271-274
std::vector<uint16_t> expect_w8a8(const std::vector<int8_t>& a, const std::vector<int8_t>& w, bool w_is_nk,
                                  const std::vector<float>& sa, const std::vector<float>& sb, int m, int n, int k) {
    std::vector<uint16_t> out(static_cast<size_t>(m) * n);
    for (int r = 0; r < m; ++r) {
        for (int j = 0; j < n; ++j) {
            int32_t acc = 0;
            for (int t = 0; t < k; ++t) {
                const int8_t wv = w_is_nk ? w[static_cast<size_t>(j) * k + t] : w[static_cast<size_t>(t) * n + j];
                acc += static_cast<int32_t>(a[static_cast<size_t>(r) * k + t]) * wv;
            }
            out[static_cast<size_t>(r) * n + j] = bf16_rne((sa[r] * sb[j]) * static_cast<float>(acc));
        }
    }
    return out;
}

// the per-token quantiser of the decode step: scale = absmax / 127 (1 if the row is zero), q = clamp(rint(x * (1/scale)))
// (crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:160-200)
void quantize_row(const std::vector<uint16_t>& x_bf16, int k, std::vector<int8_t>& q, float& scale) {
    float amax = 0.0f;
    for (int t = 0; t < k; ++t) amax = std::fmax(amax, std::fabs(bf16_to_f32(x_bf16[t])));
    scale = amax > 0.0f ? amax / 127.0f : 1.0f;
    const float inv = 1.0f / scale;
    q.resize(k);
    for (int t = 0; t < k; ++t) {
        float v = std::nearbyintf(bf16_to_f32(x_bf16[t]) * inv);
        v = std::fmin(std::fmax(v, -127.0f), 127.0f);
        q[t] = static_cast<int8_t>(v);
    }
}

template <typename T>
T* to_device(const std::vector<T>& v) {
    T* p = nullptr;
    if (cudaMalloc(&p, v.size() * sizeof(T)) != cudaSuccess) return nullptr;
    if (cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
    return p;
}

struct Graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

}  // namespace

int main() {
    int ndev = 0;
    CK(cudaGetDeviceCount(&ndev));
    REQUIRE(ndev > 0);
    CK(cudaSetDevice(0));
    cudaStream_t stream;
    CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    uint32_t seed = 12345u;

    // ---- decode GEMV, K = 4096, N = 14336, m = 1, both weight layouts -------------------------------------------
    const int k = 4096, n = 14336;
    std::vector<int8_t> w(static_cast<size_t>(n) * k);
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(lcg(seed) % 255u) - 127);
    std::vector<float> sb(n), sa(1);
    for (auto& v : sb) v = 0.0005f + static_cast<float>(lcg(seed) % 1000u) * 1e-6f;
    std::vector<int8_t> x0(k), x1(k);
    for (auto& v : x0) v = static_cast<int8_t>(static_cast<int>(lcg(seed) % 255u) - 127);
    for (auto& v : x1) v = static_cast<int8_t>(static_cast<int>(lcg(seed) % 255u) - 127);
    sa[0] = 0.0123f;
    int8_t* d_w = to_device(w);
    float* d_sb = to_device(sb);
    float* d_sa = to_device(sa);
    int8_t* d_x = to_device(x0);
    REQUIRE(d_w && d_sb && d_sa && d_x);
    uint16_t* d_out = nullptr;
    CK(cudaMalloc(&d_out, static_cast<size_t>(n) * 2));
    std::vector<uint16_t> got(n);

    for (int layout = 1; layout >= 0; --layout) {  // 1: weights [N,K]; 0: the same bytes read as row-major [K,N]
        const int nn = layout == 1 ? n : k, kk = layout == 1 ? k : n;  // [14336,4096] bytes = [K=14336, N=4096] row-major
        const int64_t ldb = layout == 1 ? kk : nn;
        std::vector<int8_t> xa(kk), xb(kk);
        for (int t = 0; t < kk; ++t) {
            xa[t] = x0[t % k];
            xb[t] = x1[(t * 7) % k];
        }
        int8_t* d_xx = to_device(xa);
        REQUIRE(d_xx);
        const auto want_a = expect_w8a8(xa, w, layout == 1, sa, sb, 1, nn, kk);
        const auto want_b = expect_w8a8(xb, w, layout == 1, sa, sb, 1, nn, kk);
        REQUIRE(baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement(1, nn, kk, 1, layout, kk, ldb, nn, 0, 0, 0) == 0);
        const size_t ws_bytes = baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(1, nn, kk, 1, layout);
        void* d_ws = nullptr;
        if (ws_bytes) CK(cudaMalloc(&d_ws, ws_bytes));
        auto call = [&](cudaStream_t s) {
            return baracuda_kernels_gemv_q8_m1_bf16_sm100a_run(1, nn, kk, 1, layout, 1.0f, 0.0f, d_xx, kk, 0, d_w, ldb, 0,
                                                               d_sa, 0, d_sb, 0, d_out, nn, 0, d_ws, ws_bytes, s);
        };
        CK(cudaMemset(d_out, 0, static_cast<size_t>(n) * 2));
        REQUIRE(call(stream) == 0);  // eager warm launch
        CK(cudaStreamSynchronize(stream));
        CK(cudaMemcpy(got.data(), d_out, static_cast<size_t>(nn) * 2, cudaMemcpyDeviceToHost));
        REQUIRE(std::memcmp(got.data(), want_a.data(), static_cast<size_t>(nn) * 2) == 0);

        Graph g;
        CK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeGlobal));
        const int32_t st = call(stream);  // an allocation or a synchronisation in here would invalidate the capture
        CK(cudaStreamEndCapture(stream, &g.graph));
        REQUIRE(st == 0);
        CK(cudaGraphInstantiate(&g.exec, g.graph, 0));
        for (int rep = 0; rep < 3; ++rep) {  // replay on the warm result, no re-zeroing
            CK(cudaGraphLaunch(g.exec, stream));
            CK(cudaStreamSynchronize(stream));
            CK(cudaMemcpy(got.data(), d_out, static_cast<size_t>(nn) * 2, cudaMemcpyDeviceToHost));
            REQUIRE(std::memcmp(got.data(), want_a.data(), static_cast<size_t>(nn) * 2) == 0);
        }
        CK(cudaMemcpy(d_xx, xb.data(), kk, cudaMemcpyHostToDevice));  // new token, same graph
        CK(cudaGraphLaunch(g.exec, stream));
        CK(cudaStreamSynchronize(stream));
        CK(cudaMemcpy(got.data(), d_out, static_cast<size_t>(nn) * 2, cudaMemcpyDeviceToHost));
        REQUIRE(std::memcmp(got.data(), want_b.data(), static_cast<size_t>(nn) * 2) == 0);
        CK(cudaGraphExecDestroy(g.exec));
        CK(cudaGraphDestroy(g.graph));
        CK(cudaFree(d_xx));
        if (d_ws) CK(cudaFree(d_ws));
    }

    // ---- the whole decode step (per-token quantiser + GEMV) from bf16 activations in one captured launch ----------
    {
        std::vector<uint16_t> xh(k), xh2(k);
        for (int t = 0; t < k; ++t) {
            xh[t] = bf16_rne((static_cast<float>(lcg(seed) % 2001u) - 1000.0f) * 0.003f);
            xh2[t] = bf16_rne((static_cast<float>(lcg(seed) % 2001u) - 1000.0f) * 0.0007f);
        }
        uint16_t* d_xh = to_device(xh);
        float* d_qs = nullptr;
        CK(cudaMalloc(&d_qs, 4));
        REQUIRE(d_xh);
        if (baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement(1, n, k, k, k, n) == 0) {
            auto call = [&](cudaStream_t s) {
                return baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_run(1, n, k, -127, 127, 1.0f, 0.0f, d_xh, k, d_w, k,
                                                                              d_sb, d_qs, d_out, n, nullptr, 0, s);
            };
            Graph g;
            CK(cudaMemset(d_out, 0, static_cast<size_t>(n) * 2));
            REQUIRE(call(stream) == 0);
            CK(cudaStreamSynchronize(stream));
            CK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeGlobal));
            const int32_t st = call(stream);
            CK(cudaStreamEndCapture(stream, &g.graph));
            REQUIRE(st == 0);
            CK(cudaGraphInstantiate(&g.exec, g.graph, 0));
            for (int rep = 0; rep < 2; ++rep) {
                const std::vector<uint16_t>& cur = rep == 0 ? xh : xh2;
                CK(cudaMemcpy(d_xh, cur.data(), static_cast<size_t>(k) * 2, cudaMemcpyHostToDevice));
                CK(cudaGraphLaunch(g.exec, stream));
                CK(cudaStreamSynchronize(stream));
                std::vector<int8_t> q;
                std::vector<float> s1(1);
                quantize_row(cur, k, q, s1[0]);
                const auto want = expect_w8a8(q, w, true, s1, sb, 1, n, k);
                CK(cudaMemcpy(got.data(), d_out, static_cast<size_t>(n) * 2, cudaMemcpyDeviceToHost));
                REQUIRE(std::memcmp(got.data(), want.data(), static_cast<size_t>(n) * 2) == 0);
                float s_dev = 0.0f;
                CK(cudaMemcpy(&s_dev, d_qs, 4, cudaMemcpyDeviceToHost));
                REQUIRE(s_dev == s1[0]);  // the activation scale is handed back
            }
            CK(cudaGraphExecDestroy(g.exec));
            CK(cudaGraphDestroy(g.graph));
        } else {
            std::printf("one-launch decode step declined this shape\n");
            return 1;
        }
    }

    // ---- W8A8 GEMM 128 x 1024 x 1024 (tensor maps are kernel parameters: captured by value) -----------------------
    {
        const int m = 128, gn = 1024, gk = 1024;
        std::vector<int8_t> a(static_cast<size_t>(m) * gk), a2(a.size());
        for (auto& v : a) v = static_cast<int8_t>(static_cast<int>(lcg(seed) % 255u) - 127);
        for (auto& v : a2) v = static_cast<int8_t>(static_cast<int>(lcg(seed) % 255u) - 127);
        std::vector<int8_t> gw(w.begin(), w.begin() + static_cast<size_t>(gn) * gk);
        std::vector<float> gsa(m), gsb(sb.begin(), sb.begin() + gn);
        for (auto& v : gsa) v = 0.002f + static_cast<float>(lcg(seed) % 1000u) * 1e-5f;
        int8_t* d_a = to_device(a);
        float* d_gsa = to_device(gsa);
        uint16_t* d_y = nullptr;
        CK(cudaMalloc(&d_y, static_cast<size_t>(m) * gn * 2));
        REQUIRE(d_a && d_gsa);
        auto call = [&](cudaStream_t s) {
            return baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run(m, gn, gk, d_a, gk, d_w, gk, nullptr, 0, d_y, gn, d_gsa,
                                                                     d_sb, 1.0f, 0.0f, nullptr, 0, s);
        };
        CK(cudaMemset(d_y, 0, static_cast<size_t>(m) * gn * 2));
        REQUIRE(call(stream) == 0);
        CK(cudaStreamSynchronize(stream));
        Graph g;
        CK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeGlobal));
        const int32_t st = call(stream);
        CK(cudaStreamEndCapture(stream, &g.graph));
        REQUIRE(st == 0);
        CK(cudaGraphInstantiate(&g.exec, g.graph, 0));
        std::vector<uint16_t> y(static_cast<size_t>(m) * gn);
        for (int rep = 0; rep < 2; ++rep) {
            const std::vector<int8_t>& cur = rep == 0 ? a : a2;
            CK(cudaMemcpy(d_a, cur.data(), cur.size(), cudaMemcpyHostToDevice));
            CK(cudaGraphLaunch(g.exec, stream));
            CK(cudaStreamSynchronize(stream));
            const auto want = expect_w8a8(cur, gw, true, gsa, gsb, m, gn, gk);
            CK(cudaMemcpy(y.data(), d_y, y.size() * 2, cudaMemcpyDeviceToHost));
            REQUIRE(std::memcmp(y.data(), want.data(), y.size() * 2) == 0);
        }
        CK(cudaGraphExecDestroy(g.exec));
        CK(cudaGraphDestroy(g.graph));
    }

    // ---- the C++ Plan layer: two decode steps chained as programmatic dependent launches in ONE graph, then SmoothQuant --
    {
        using namespace baracuda;
        PlanPreference pref;
        QuantizedLinearDescriptor ld;
        ld.m = 1;
        ld.c_out = n;
        ld.k = k;
        QuantizedLinearPlan ql;
        REQUIRE(QuantizedLinearPlan::select(ld, pref, &ql) == Error::Ok);
        std::vector<uint16_t> xh(k);
        for (int t = 0; t < k; ++t) xh[t] = bf16_rne((static_cast<float>(lcg(seed) % 2001u) - 1000.0f) * 0.002f);
        uint16_t* d_xh = to_device(xh);
        REQUIRE(d_xh);
        float* d_qs = nullptr;
        int8_t* d_q = nullptr;
        uint16_t* d_out2 = nullptr;
        CK(cudaMalloc(&d_qs, 4));
        CK(cudaMalloc(&d_q, k));
        CK(cudaMalloc(&d_out2, static_cast<size_t>(n) * 2));
        QuantizedLinearArgs la;
        la.activation = {d_xh, static_cast<size_t>(k)};
        la.weight_q = {d_w, static_cast<size_t>(n) * k};
        la.weight_scale = {d_sb, static_cast<size_t>(n)};
        la.output = {d_out, static_cast<size_t>(n)};
        la.act_q_scratch = {d_q, static_cast<size_t>(k)};
        la.act_scale_scratch = {d_qs, 1};
        REQUIRE(ql.fused_decode(la));
        QuantizedLinearArgs lb = la;
        lb.output = {d_out2, static_cast<size_t>(n)};
        void* d_ws = nullptr;
        const size_t ws_bytes = ql.workspace_size();
        if (ws_bytes) CK(cudaMalloc(&d_ws, ws_bytes));
        CK(cudaMemset(d_out, 0, static_cast<size_t>(n) * 2));
        CK(cudaMemset(d_out2, 0, static_cast<size_t>(n) * 2));
        Graph g;
        CK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeGlobal));
        const Error e1 = ql.run(stream, Workspace{d_ws, ws_bytes}, la, false);
        const Error e2 = ql.run(stream, Workspace{d_ws, ws_bytes}, lb, true);  // prefetches weights while the first drains
        CK(cudaStreamEndCapture(stream, &g.graph));
        REQUIRE(e1 == Error::Ok && e2 == Error::Ok);
        CK(cudaGraphInstantiate(&g.exec, g.graph, 0));
        std::vector<int8_t> q;
        std::vector<float> s1(1);
        quantize_row(xh, k, q, s1[0]);
        const auto want = expect_w8a8(q, w, true, s1, sb, 1, n, k);
        for (int rep = 0; rep < 2; ++rep) {
            CK(cudaGraphLaunch(g.exec, stream));
            CK(cudaStreamSynchronize(stream));
            CK(cudaMemcpy(got.data(), d_out, static_cast<size_t>(n) * 2, cudaMemcpyDeviceToHost));
            REQUIRE(std::memcmp(got.data(), want.data(), static_cast<size_t>(n) * 2) == 0);
            CK(cudaMemcpy(got.data(), d_out2, static_cast<size_t>(n) * 2, cudaMemcpyDeviceToHost));
            REQUIRE(std::memcmp(got.data(), want.data(), static_cast<size_t>(n) * 2) == 0);
        }
        CK(cudaGraphExecDestroy(g.exec));
        CK(cudaGraphDestroy(g.graph));

        // SmoothQuant: one per-tensor activation scale by value; the same bits as the per-token kernel on a constant vector
        const int m = 128, gn = 1024, gk = 1024;
        SmoothQuantLinearDescriptor sd;
        sd.m = m;
        sd.n = gn;
        sd.k = gk;
        sd.act_scale = 0.0173f;
        SmoothQuantLinearPlan sq;
        REQUIRE(SmoothQuantLinearPlan::select(sd, pref, &sq) == Error::Ok);
        std::vector<int8_t> a(static_cast<size_t>(m) * gk);
        for (auto& v : a) v = static_cast<int8_t>(static_cast<int>(lcg(seed) % 255u) - 127);
        std::vector<int8_t> gw(w.begin(), w.begin() + static_cast<size_t>(gn) * gk);
        std::vector<float> gsa(m, sd.act_scale), gsb(sb.begin(), sb.begin() + gn);
        int8_t* d_a = to_device(a);
        uint16_t* d_y = nullptr;
        CK(cudaMalloc(&d_y, static_cast<size_t>(m) * gn * 2));
        REQUIRE(d_a);
        SmoothQuantLinearArgs sx;
        sx.act_q = {d_a, a.size()};
        sx.weight_q = {d_w, gw.size()};
        sx.weight_scale = {d_sb, static_cast<size_t>(gn)};
        sx.output = {d_y, static_cast<size_t>(m) * gn};
        REQUIRE(sq.run(stream, Workspace::none(), sx) == Error::Ok);
        CK(cudaStreamSynchronize(stream));
        std::vector<uint16_t> y(static_cast<size_t>(m) * gn);
        CK(cudaMemcpy(y.data(), d_y, y.size() * 2, cudaMemcpyDeviceToHost));
        const auto want_sq = expect_w8a8(a, gw, true, gsa, gsb, m, gn, gk);
        REQUIRE(std::memcmp(y.data(), want_sq.data(), y.size() * 2) == 0);
    }

    REQUIRE(baracuda_kernels_q_device_status() == 0);
    std::printf("capture_replay_host ok\n");
    return 0;
}
