// A compiled host for the decode projection set: what a native caller of the C ABI sees end to end.
//
// Per step, through include/tessl_b200.h only: three activation vectors written from pinned host
// memory, four operator calls (q/k/v as one bank, o_proj, fused gate/up + SiLU with a bf16 result,
// down), and the down projection's output read back to pinned host memory. Timed with the host
// clock around `steps` such steps, once with every call synchronous (the ABI's default) and once in
// encode-only mode, where only the read waits. The banks are the seeded synthetic ones of
// tessl_b200/synth.py (same splitmix64 stream and formulas, so layer 0 here is bit for bit the bank a
// Python caller builds from the same seed); the step rotates over `layers` layers so that the
// weight stream does not fit L2.
//
//   tessl_step_driver [--steps K] [--warmup W] [--layers L] [--seed S] [--device D] [--y-out FILE]
//
// Prints one JSON object. With --y-out, the first step's result (layer 0) is written as raw f32.
#include <cuda_runtime_api.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/tessl_b200.h"

namespace {

constexpr uint32_t kHidden = 4096, kQkv = 6144, kInter = 12288, kGroup = 64;
constexpr uint64_t kGamma = 0x9E3779B97F4A7C15ull;

[[noreturn]] void die(const std::string &what)
{
    std::fprintf(stderr, "tessl_step_driver: %s\n", what.c_str());
    std::exit(1);
}

char g_err[1024];
void must(int32_t st, const char *what)
{
    if (st != TESSL_OK) die(std::string(what) + ": " + g_err);
}

// Draw i (from 1) of the stream seeded with `seed`: state seed ^ GAMMA advanced i times, then mixed.
inline uint64_t draw(uint64_t seed, uint64_t i)
{
    uint64_t z = (seed ^ kGamma) + i * kGamma;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
inline double uniform01(uint64_t d) { return ((double)(d >> 40) + 0.5) / 16777216.0; }
inline uint16_t bf16_bits(float f)
{
    uint32_t b;
    std::memcpy(&b, &f, 4);
    return (uint16_t)(((uint64_t)b + 0x7FFF + ((b >> 16) & 1)) >> 16);
}
inline float bf16_value(uint16_t h)
{
    const uint32_t b = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}

struct HostBank {
    std::vector<uint32_t> packed;
    std::vector<uint16_t> pairs;
};

// tessl_b200/synth.py `q4_bank`: nibbles = top four bits of a draw, eight per little-endian word;
// scale ~ U(0.002, 0.02), bias = -8 * scale + N(0, 0.001), both bf16, stored as adjacent pairs.
HostBank q4_bank(uint64_t seed, uint32_t rows, uint32_t cols)
{
    HostBank b;
    const uint64_t words = (uint64_t)rows * cols / 8, groups = (uint64_t)rows * (cols / kGroup);
    b.packed.resize(words);
    b.pairs.resize(2 * groups);
    auto fill = [&](uint64_t w0, uint64_t w1) {
        for (uint64_t w = w0; w < w1; ++w) {
            uint32_t v = 0;
            for (uint32_t i = 0; i < 8; ++i) v |= (uint32_t)(draw(seed, 8 * w + i + 1) >> 60) << (4 * i);
            b.packed[w] = v;
        }
    };
    const unsigned nt = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < nt; ++t) pool.emplace_back(fill, words * t / nt, words * (t + 1) / nt);
    for (auto &t : pool) t.join();
    const double two_pi = 2.0 * 3.141592653589793;
    for (uint64_t g = 0; g < groups; ++g) {
        const double u = uniform01(draw(seed + 1, g + 1));
        const uint16_t s = bf16_bits((float)(0.002 + u * (0.02 - 0.002)));
        const double u1 = uniform01(draw(seed + 1, groups + g + 1)), u2 = uniform01(draw(seed + 1, 2 * groups + g + 1));
        const double noise = std::sqrt(-2.0 * std::log(u1)) * std::cos(two_pi * u2) * 0.001;
        b.pairs[2 * g] = s;
        b.pairs[2 * g + 1] = bf16_bits((float)(-8.0 * (double)bf16_value(s) + noise));
    }
    return b;
}

// tessl_b200/synth.py `normal_bf16`: Box-Muller over pairs of draws, rounded to bf16.
std::vector<uint16_t> normal_bf16(uint64_t seed, uint32_t n)
{
    std::vector<uint16_t> out(n);
    const double two_pi = 2.0 * 3.141592653589793;
    for (uint32_t p = 0; 2 * p < n; ++p) {
        const double u1 = uniform01(draw(seed, 2 * p + 1)), u2 = uniform01(draw(seed, 2 * p + 2));
        const double r = std::sqrt(-2.0 * std::log(u1));
        out[2 * p] = bf16_bits((float)(r * std::cos(two_pi * u2)));
        if (2 * p + 1 < n) out[2 * p + 1] = bf16_bits((float)(r * std::sin(two_pi * u2)));
    }
    return out;
}

struct Layer {
    TesslQ4MlxBank qkv, o, gate, up, down;
};

TesslQ4MlxBank upload(TesslRuntime *rt, const HostBank &h)
{
    TesslQ4MlxBank b{};
    must(tessl_buffer_alloc(rt, h.packed.size() * 4, &b.packed, g_err, sizeof g_err), "alloc packed");
    must(tessl_buffer_alloc(rt, h.pairs.size() * 2, &b.scales_biases, g_err, sizeof g_err), "alloc pairs");
    must(tessl_buffer_write(rt, b.packed, 0, h.packed.data(), h.packed.size() * 4, g_err, sizeof g_err), "write packed");
    must(tessl_buffer_write(rt, b.scales_biases, 0, h.pairs.data(), h.pairs.size() * 2, g_err, sizeof g_err), "write pairs");
    return b;
}

uint64_t bank_bytes(uint32_t rows, uint32_t cols) { return (uint64_t)rows * cols / 2 + (uint64_t)rows * (cols / kGroup) * 4; }

template <typename T>
T *pinned(size_t n)
{
    void *p = nullptr;
    if (cudaHostAlloc(&p, n * sizeof(T), cudaHostAllocDefault) != cudaSuccess) die("cudaHostAlloc failed");
    return static_cast<T *>(p);
}

}  // namespace

int main(int argc, char **argv)
{
    int steps = 200, warmup = 5, layers = 4, device = 0;
    uint64_t seed = 0x7E550100ull;
    std::string y_out;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&]() -> const char * {
            if (i + 1 >= argc) die("missing value after " + a);
            return argv[++i];
        };
        if (a == "--steps") steps = std::atoi(next());
        else if (a == "--warmup") warmup = std::atoi(next());
        else if (a == "--layers") layers = std::atoi(next());
        else if (a == "--device") device = std::atoi(next());
        else if (a == "--seed") seed = std::strtoull(next(), nullptr, 0);
        else if (a == "--y-out") y_out = next();
        else die("unknown argument " + a);
    }
    if (steps < 1 || warmup < 0 || layers < 1 || layers > 16) die("steps >= 1, warmup >= 0, 1 <= layers <= 16");
    if (tessl_abi_version() != TESSL_B200_ABI_VERSION) die("library ABI differs from the header");

    TesslRuntime *rt = tessl_runtime_new_on_device(device, g_err, sizeof g_err);
    if (!rt) die(std::string("tessl_runtime_new_on_device: ") + g_err);

    // layer l's banks use seed + 0x1000 * l + 16 * {0: qkv, 1: o, 2: gate, 3: up, 4: down}
    std::vector<Layer> L(layers);
    for (int l = 0; l < layers; ++l) {
        const uint64_t s = seed + 0x1000ull * l;
        L[l].qkv = upload(rt, q4_bank(s, kQkv, kHidden));
        L[l].o = upload(rt, q4_bank(s + 16, kHidden, kHidden));
        L[l].gate = upload(rt, q4_bank(s + 32, kInter, kHidden));
        L[l].up = upload(rt, q4_bank(s + 48, kInter, kHidden));
        L[l].down = upload(rt, q4_bank(s + 64, kHidden, kInter));
    }
    uint16_t *hx[3];
    TesslBuf dx[3];
    for (int i = 0; i < 3; ++i) {
        const std::vector<uint16_t> x = normal_bf16(seed + 1000 + i, kHidden);
        hx[i] = pinned<uint16_t>(kHidden);
        std::memcpy(hx[i], x.data(), kHidden * 2);
        must(tessl_buffer_alloc(rt, kHidden * 2, &dx[i], g_err, sizeof g_err), "alloc x");
    }
    TesslBuf qkv_out, o_out, mid, y;
    must(tessl_buffer_alloc(rt, kQkv * 4, &qkv_out, g_err, sizeof g_err), "alloc qkv_out");
    must(tessl_buffer_alloc(rt, kHidden * 4, &o_out, g_err, sizeof g_err), "alloc o_out");
    must(tessl_buffer_alloc(rt, kInter * 2, &mid, g_err, sizeof g_err), "alloc mid");
    must(tessl_buffer_alloc(rt, kHidden * 4, &y, g_err, sizeof g_err), "alloc y");
    float *hy = pinned<float>(kHidden);

    const TesslQuantShape sq{kQkv, kHidden, kGroup}, so{kHidden, kHidden, kGroup}, sg{kInter, kHidden, kGroup},
        sd{kHidden, kInter, kGroup};
    auto step = [&](int i) {
        const Layer &l = L[i % layers];
        for (int k = 0; k < 3; ++k) must(tessl_buffer_write(rt, dx[k], 0, hx[k], kHidden * 2, g_err, sizeof g_err), "write x");
        must(tessl_gemv_q4_mlx_simd(rt, l.qkv, dx[0], qkv_out, sq, TESSL_Q4_ROW_MAJOR, nullptr, g_err, sizeof g_err), "qkv");
        must(tessl_gemv_q4_mlx_simd(rt, l.o, dx[1], o_out, so, TESSL_Q4_ROW_MAJOR, nullptr, g_err, sizeof g_err), "o");
        must(tessl_gemv_q4_mlx_gate_up_silu(rt, l.gate, l.up, dx[2], mid, sg, 1, g_err, sizeof g_err), "gate_up_silu");
        must(tessl_gemv_q4_mlx_simd(rt, l.down, mid, y, sd, TESSL_Q4_ROW_MAJOR, nullptr, g_err, sizeof g_err), "down");
        must(tessl_buffer_read(rt, y, 0, hy, kHidden * 4, g_err, sizeof g_err), "read y");
    };

    step(0);
    if (!y_out.empty()) {
        FILE *f = std::fopen(y_out.c_str(), "wb");
        if (!f || std::fwrite(hy, 4, kHidden, f) != kHidden) die("cannot write " + y_out);
        std::fclose(f);
    }
    double checksum = 0.0;
    for (uint32_t i = 0; i < kHidden; ++i) checksum += (double)hy[i];

    auto timed = [&]() {
        for (int i = 0; i < std::max(warmup, 3); ++i) step(i);
        must(tessl_synchronize(rt, g_err, sizeof g_err), "synchronize");
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < steps; ++i) step(i);
        must(tessl_synchronize(rt, g_err, sizeof g_err), "synchronize");
        return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / steps;
    };
    const double ms_sync = timed();
    must(tessl_runtime_set_encode_only(rt, 1, g_err, sizeof g_err), "encode-only on");
    const double ms = timed();
    must(tessl_runtime_set_encode_only(rt, 0, g_err, sizeof g_err), "encode-only off");
    uint64_t launches = 0;
    must(tessl_runtime_take_dispatch_count(rt, &launches, g_err, sizeof g_err), "dispatch count");

    const uint64_t step_bytes = bank_bytes(kQkv, kHidden) + bank_bytes(kHidden, kHidden) + 2 * bank_bytes(kInter, kHidden) +
                                bank_bytes(kHidden, kInter);
    std::printf("{\"host\": \"compiled C++ over the C ABI\", \"steps\": %d, \"layers\": %d, \"ms_per_step\": %.6f, "
                "\"ms_per_step_synchronous\": %.6f, \"value\": %.2f, \"value_every_call_synchronous\": %.2f, "
                "\"unit\": \"GB/s\", \"h2d_bytes_per_step\": %u, \"d2h_bytes_per_step\": %u, \"weight_bytes_per_step\": %llu, "
                "\"y_checksum\": %.9g}\n",
                steps, layers, ms, ms_sync, step_bytes / (ms * 1e-3) / 1e9, step_bytes / (ms_sync * 1e-3) / 1e9, 3 * kHidden * 2,
                kHidden * 4, (unsigned long long)step_bytes, checksum);
    (void)launches;
    tessl_runtime_free(rt);
    return 0;
}
