// Torch-free driver for the native launchers of libi8tk_compat.so: links them by their C++
// names the way the reference's own CUDA test does (tests/cuda/test_int8.cu:15-26), runs each
// one on seeded inputs and compares with the C ABI (i8tk.h) called on the same inputs with a
// caller-owned workspace.  Both routes run the same kernels, so the comparison is bit for bit.
// Prints one line per case and "ALL OK" at the end; the exit code is the number of failures.
// With the argument "link-only" it makes no CUDA call (used where there is no GPU).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../include/i8tk.h"
#include "../include/i8tk_compat.h"

namespace {

uint32_t g_seed = 12345u;
uint32_t rnd() { g_seed = g_seed * 1664525u + 1013904223u; return g_seed >> 8; }

template <typename T>
T* dev(const std::vector<T>& h) {
    T* p = nullptr;
    cudaMalloc(reinterpret_cast<void**>(&p), h.size() * sizeof(T) + 256);
    cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return p;
}
template <typename T>
T* dev_empty(size_t n) {
    T* p = nullptr;
    cudaMalloc(reinterpret_cast<void**>(&p), n * sizeof(T) + 256);
    cudaMemset(p, 0xA5, n * sizeof(T));
    return p;
}
template <typename T>
bool same(const T* a, const T* b, size_t n) {
    std::vector<T> ha(n), hb(n);
    cudaMemcpy(ha.data(), a, n * sizeof(T), cudaMemcpyDeviceToHost);
    cudaMemcpy(hb.data(), b, n * sizeof(T), cudaMemcpyDeviceToHost);
    return std::memcmp(ha.data(), hb.data(), n * sizeof(T)) == 0;
}
std::vector<int8_t> codes(size_t n) {
    std::vector<int8_t> v(n);
    for (auto& x : v) x = (int8_t)((int)(rnd() % 255u) - 127);
    return v;
}
std::vector<float> scales(size_t n, float lo, float span) {
    std::vector<float> v(n);
    for (auto& x : v) x = lo + span * (float)(rnd() % 1000u) / 1000.f;
    return v;
}

int report(const char* name, bool ok) {
    std::printf("%-44s %s (status %d)\n", name, ok ? "OK" : "MISMATCH", i8tk_compat_last_status());
    return ok ? 0 : 1;
}

int decode_case(int BH, int S, int D) {
    auto Q = dev(codes((size_t)BH * D)), K = dev(codes((size_t)BH * S * D)), V = dev(codes((size_t)BH * S * D));
    auto sQ = dev(scales(BH, 0.01f, 0.02f)), sK = dev(scales((size_t)BH * S, 0.01f, 0.02f));
    auto sV = dev(scales((size_t)BH * S, 0.01f, 0.02f));
    half* a = dev_empty<half>((size_t)BH * D);
    half* b = dev_empty<half>((size_t)BH * D);
    int8_decode_attention_forward(Q, K, V, a, sQ, sK, sV, BH, S, D);
    const bool launched = i8tk_compat_last_status() == I8TK_OK;
    const size_t wb = i8tk_decode_workspace_bytes(BH, S, D);
    void* ws = dev_empty<unsigned char>(wb);
    const int rc = i8tk_decode_attention_forward(Q, K, V, b, sQ, sK, sV, BH, S, D, ws, wb, nullptr);
    cudaDeviceSynchronize();
    char name[96];
    std::snprintf(name, sizeof(name), "int8_decode_attention_forward BH%d S%d D%d", BH, S, D);
    return report(name, launched && rc == I8TK_OK && same(a, b, (size_t)BH * D));
}

int prefill_case(int B, int H, int S, int D) {
    const size_t n = (size_t)B * H * S * D, rows = (size_t)B * H * S;
    auto Q = dev(codes(n)), K = dev(codes(n)), V = dev(codes(n));
    auto sQ = dev(scales(rows, 0.005f, 0.01f)), sK = dev(scales(rows, 0.005f, 0.01f)), sV = dev(scales(rows, 0.01f, 0.02f));
    half* a = dev_empty<half>(n);
    half* b = dev_empty<half>(n);
    int8_attention_forward(Q, K, V, a, sQ, sK, sV, B, H, S, D);
    const bool launched = i8tk_compat_last_status() == I8TK_OK;
    const size_t wb = i8tk_attention_workspace_bytes(B, H, S, D);
    void* ws = dev_empty<unsigned char>(wb);
    const int rc = i8tk_attention_forward(Q, K, V, b, sQ, sK, sV, B, H, S, D, ws, wb, nullptr);
    cudaDeviceSynchronize();
    char name[96];
    std::snprintf(name, sizeof(name), "int8_attention_forward B%d H%d S%d D%d", B, H, S, D);
    return report(name, launched && rc == I8TK_OK && same(a, b, n));
}

int mlp_cases(int batch, int seq, int dm, int dff) {
    const int T = batch * seq;
    int fails = 0;
    auto x = dev(codes((size_t)T * dm)), W1 = dev(codes((size_t)dm * dff)), W2 = dev(codes((size_t)dff * dm));
    auto sx = dev(scales(T, 0.01f, 0.02f)), s1 = dev(scales(dff, 2e-4f, 2e-4f)), s2 = dev(scales(dm, 2e-4f, 2e-4f));
    auto b1 = dev(scales(dff, -0.01f, 0.02f));
    int8_t* oa = dev_empty<int8_t>((size_t)T * dm);
    int8_t* ob = dev_empty<int8_t>((size_t)T * dm);
    float* ra = dev_empty<float>(T);
    float* rb = dev_empty<float>(T);
    float* tscale = dev_empty<float>(1);
    const size_t wb = i8tk_mlp_workspace_bytes(T, dm, dff, 7);
    void* ws = dev_empty<unsigned char>(wb);

    // per-token / per-channel, with and without the pre-GELU bias
    for (int with_bias = 0; with_bias < 2; ++with_bias) {
        if (with_bias) int8_mlp_forward_per_channel_bias(x, W1, W2, oa, sx, s1, s2, b1, ra, batch, seq, dm, dff);
        else int8_mlp_forward_per_channel(x, W1, W2, oa, sx, s1, s2, ra, batch, seq, dm, dff);
        const bool launched = i8tk_compat_last_status() == I8TK_OK;
        const int rc = i8tk_mlp_forward(x, W1, W2, ob, sx, s1, s2, with_bias ? b1 : nullptr, rb, nullptr, T, dm, dff,
                                        I8TK_MLP_X_PER_TOKEN | I8TK_MLP_W_PER_CHANNEL, ws, wb, nullptr);
        cudaDeviceSynchronize();
        fails += report(with_bias ? "int8_mlp_forward_per_channel_bias" : "int8_mlp_forward_per_channel",
                        launched && rc == I8TK_OK && same(oa, ob, (size_t)T * dm) && same(ra, rb, T));
    }
    // per-tensor scales, dynamic per-tensor output scale read back through the getter
    {
        int8_mlp_forward(x, W1, W2, oa, sx, s1, s2, batch, seq, dm, dff);
        const bool launched = i8tk_compat_last_status() == I8TK_OK;
        float got = -1.f, want = -2.f;
        int8_mlp_get_output_scale(&got);
        const int rc = i8tk_mlp_forward(x, W1, W2, ob, sx, s1, s2, nullptr, nullptr, tscale, T, dm, dff, 0, ws, wb, nullptr);
        cudaMemcpy(&want, tscale, sizeof(float), cudaMemcpyDeviceToHost);
        fails += report("int8_mlp_forward + int8_mlp_get_output_scale",
                        launched && rc == I8TK_OK && same(oa, ob, (size_t)T * dm) && got == want && got > 0.f);
    }
    // weights transposed once, then the prepacked launcher: same bytes as the call above
    {
        int8_t* W1T = dev_empty<int8_t>((size_t)dm * dff);
        int8_t* W2T = dev_empty<int8_t>((size_t)dm * dff);
        transpose_int8_weights(W1, W2, W1T, W2T, dm, dff);
        const bool t_ok = i8tk_compat_last_status() == I8TK_OK;
        int8_t* oc = dev_empty<int8_t>((size_t)T * dm);
        int8_mlp_forward_prepacked(x, W1T, W2T, oc, sx, s1, s2, batch, seq, dm, dff);
        const bool launched = i8tk_compat_last_status() == I8TK_OK;
        cudaDeviceSynchronize();
        fails += report("transpose_int8_weights + int8_mlp_forward_prepacked",
                        t_ok && launched && same(oa, oc, (size_t)T * dm));
    }
    return fails;
}

int quant_case(int n) {
    std::vector<half> h(n);
    for (auto& v : h) v = __float2half(((float)(rnd() % 2001u) - 1000.f) / 250.f);
    half* in = dev(h);
    int8_t* qa = dev_empty<int8_t>(n);
    int8_t* qb = dev_empty<int8_t>(n);
    float* sa = dev_empty<float>(1);
    float* sb = dev_empty<float>(1);
    quantize_fp16_to_int8(in, qa, sa, n);
    const bool launched = i8tk_compat_last_status() == I8TK_OK;
    const int rc = i8tk_quantize_fp16_to_int8(in, qb, sb, n, nullptr);
    float scale = 0.f;
    cudaMemcpy(&scale, sa, sizeof(float), cudaMemcpyDeviceToHost);
    half* da = dev_empty<half>(n);
    half* db = dev_empty<half>(n);
    dequantize_int8_to_fp16(qa, da, scale, n);
    const bool launched2 = i8tk_compat_last_status() == I8TK_OK;
    const int rc2 = i8tk_dequantize_int8_to_fp16(qb, db, scale, n, nullptr);
    cudaDeviceSynchronize();
    return report("quantize_fp16_to_int8 + dequantize_int8_to_fp16",
                  launched && launched2 && rc == I8TK_OK && rc2 == I8TK_OK && same(qa, qb, n) && same(sa, sb, 1) &&
                      same(da, db, n) && scale > 0.f);
}

}  // namespace

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "link-only") == 0) {
        // every launcher is referenced below, so reaching this line proves they all resolved
        std::printf("linked: i8tk %d, compat status %d\n", i8tk_version(), i8tk_compat_last_status());
        return 0;
    }
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        std::printf("no CUDA device\n");
        return 99;
    }
    int fails = 0;
    fails += decode_case(8, 700, 64);
    fails += decode_case(6, 1024, 128);
    fails += prefill_case(1, 2, 200, 64);
    fails += prefill_case(1, 2, 256, 128);
    fails += prefill_case(1, 1, 200, 256);
    fails += mlp_cases(2, 128, 256, 512);
    fails += quant_case(5000);
    // a head_dim the kernels do not take: nothing is launched, the status says so
    {
        half* o = dev_empty<half>(96);
        int8_decode_attention_forward(nullptr, nullptr, nullptr, o, nullptr, nullptr, nullptr, 1, 16, 96);
        fails += report("int8_decode_attention_forward head_dim 96 refused",
                        i8tk_compat_last_status() == I8TK_ERR_UNSUPPORTED);
    }
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        std::printf("CUDA error at the end: %s\n", cudaGetErrorString(e));
        ++fails;
    }
    std::printf(fails ? "%d FAILED\n" : "ALL OK\n", fails);
    return fails;
}
