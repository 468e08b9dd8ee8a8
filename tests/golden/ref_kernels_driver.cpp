// Runs a tiny Llama through the reference project's own GPU kernel bodies on the CPU.
//
// The reference keeps its kernel bodies in one plain-C header shared by its CUDA and Metal
// back ends (crates/bc-infer/src/gpu/kernels.h); the includer supplies a prelude of types,
// math and warp primitives (crates/bc-infer/src/gpu/cuda.cu:5-72 does so for CUDA).  This
// file supplies such a prelude for a host compiler: a warp is 32 OS threads that meet at a
// barrier, and WSUM / WMAX are the butterfly over xor 16, 8, 4, 2, 1 of cuda.cu:46-56.  The
// header itself is not copied here: it is taken from the reference checkout at compile
// time (-I <reference>/crates/bc-infer/src/gpu).
//
// The launch order per layer restates crates/bc-infer/src/gpu/mod.rs:454-491 and, for the
// scores, mod.rs:499-508.  Input and output are flat little-endian files written and read
// by make_golden.py.
#include <barrier>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#define uchar bc_uchar
#define ushort bc_ushort
#define uint bc_uint
#define ulong bc_ulong
typedef unsigned char uchar;
typedef unsigned short ushort;
typedef unsigned int uint;
typedef unsigned long long ulong;
struct alignas(16) float4 { float x, y, z, w; };
static inline float4 make_f4(float a, float b, float c, float d) { float4 v{a, b, c, d}; return v; }
#define F4(a, b, c, d) make_f4((a), (b), (c), (d))
#define GLOBAL
#define LOCAL
#define PRIV
#define DEVFN static inline
static inline float bits_to_float(uint b) { float f; std::memcpy(&f, &b, 4); return f; }
#define BITS2F(b) bits_to_float((uint)(b))
#define NEG_INF (-INFINITY)
static inline float half_to_float(uint h) {
    uint s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023;
    float sign = s ? -1.f : 1.f;
    if (e == 0) return sign * std::ldexp((float)m, -24);
    if (e == 31) return m ? NAN : sign * INFINITY;
    return sign * std::ldexp((float)(m | 1024), (int)e - 25);
}
#define H2F(h) half_to_float(h)
#define POPC(x) __builtin_popcount(x)

static std::barrier<> g_bar(32);
static float g_slots[32];
static thread_local uint t_lane;
static inline float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) {
        g_slots[t_lane] = v;
        g_bar.arrive_and_wait();
        float w = g_slots[t_lane ^ o];
        g_bar.arrive_and_wait();
        v += w;
    }
    return v;
}
static inline float warp_max(float v) {
    for (int o = 16; o > 0; o >>= 1) {
        g_slots[t_lane] = v;
        g_bar.arrive_and_wait();
        float w = g_slots[t_lane ^ o];
        g_bar.arrive_and_wait();
        v = v > w ? v : w;
    }
    return v;
}
#define WSUM(v) warp_sum(v)
#define WMAX(v) warp_max(v)
#define BARRIER() g_bar.arrive_and_wait()
#define SQRT(x) std::sqrt(x)
#define EXP(x) std::exp(x)
#define SIN(x) std::sin(x)
#define COS(x) std::cos(x)

#include "kernels.h"

// One "warp": every lane runs the same body, as the hardware would.
template <class F> static void warp(F body) {
    std::vector<std::thread> lanes;
    for (uint l = 0; l < 32; l++) lanes.emplace_back([=] { t_lane = l; body(l); });
    for (auto& t : lanes) t.join();
}

static std::vector<float> product(const std::vector<float>& w, const std::vector<float>& x, uint rows, uint cols, uint n) {
    // k_matmul over its grid (mod.rs:172-177): every weight row, input rows in groups of NB.
    std::vector<float> out((size_t)n * rows);
    for (uint i0 = 0; i0 < n; i0 += NB)
        for (uint r = 0; r < rows; r++)
            warp([&](uint l) { matmul((const uchar*)w.data(), x.data(), out.data(), T_F32, rows, cols, n, cols * 4, r, i0, l); });
    return out;
}

static std::vector<float> norm(const std::vector<float>& x, const std::vector<float>& w, uint cols, float eps, uint n) {
    std::vector<float> out(x.size());
    for (uint r = 0; r < n; r++) warp([&](uint l) { rms_norm(x.data(), w.data(), out.data(), cols, eps, r, l); });
    return out;
}

int main(int argc, char** argv) {
    if (argc != 3) { std::fprintf(stderr, "usage: %s <input> <output>\n", argv[0]); return 2; }
    FILE* f = std::fopen(argv[1], "rb");
    if (!f) { std::perror(argv[1]); return 1; }
    int hdr[9];
    float eps;
    if (std::fread(hdr, 4, 9, f) != 9 || std::fread(&eps, 4, 1, f) != 1) return 1;
    const uint L = hdr[0], E = hdr[1], H = hdr[2], G = hdr[3], D = hdr[4], F = hdr[5], V = hdr[6], T = hdr[7], neox = hdr[8];
    auto read = [&](size_t n) { std::vector<float> v(n); if (std::fread(v.data(), 4, n, f) != n) { std::fprintf(stderr, "short input\n"); std::exit(1); } return v; };
    std::vector<float> inv_freq = read(D / 2);
    std::vector<int> tokens(T);
    if (std::fread(tokens.data(), 4, T, f) != T) return 1;
    std::vector<float> table = read((size_t)V * E);
    const uint qd = H * D, kvd = G * D;

    // Embedding rows (model.rs:270-280), then positions 0..T of a line (model.rs:411-414).
    std::vector<float> x((size_t)T * E);
    for (uint i = 0; i < T; i++) std::memcpy(&x[(size_t)i * E], &table[(size_t)tokens[i] * E], E * 4);
    std::vector<uint> positions(T);
    for (uint i = 0; i < T; i++) positions[i] = i;
    uint masks[2] = {0, 0};
    static float sh[TILE];

    for (uint l = 0; l < L; l++) {
        std::vector<float> attn_norm = read(E), wq = read((size_t)qd * E), wk = read((size_t)kvd * E), wv = read((size_t)kvd * E),
                           wo = read((size_t)E * qd), ffn_norm = read(E), gate = read((size_t)F * E), up = read((size_t)F * E),
                           down = read((size_t)E * F);
        std::vector<float> n = norm(x, attn_norm, E, eps, T);
        std::vector<float> q = product(wq, n, qd, E, T), k = product(wk, n, kvd, E, T), v = product(wv, n, kvd, E, T);
        for (uint idx = 0; idx < T * H * (D / 2); idx++) rope(q.data(), inv_freq.data(), positions.data(), H, D, D, neox, idx);
        for (uint idx = 0; idx < T * G * (D / 2); idx++) rope(k.data(), inv_freq.data(), positions.data(), G, D, D, neox, idx);
        std::vector<float> kc((size_t)T * kvd), vc((size_t)T * kvd);
        for (uint i = 0; i < T * kvd; i++) { copy(k.data(), kc.data(), 0, T * kvd, i); copy(v.data(), vc.data(), 0, T * kvd, i); }
        std::vector<float> att((size_t)T * qd);
        for (uint r = 0; r < T; r++)
            for (uint h = 0; h < H; h++)
                warp([&](uint lane) { attention(q.data(), kc.data(), vc.data(), att.data(), sh, masks, 0, H, G, D, 0, 1.0f / std::sqrt((float)D), h, r, lane); });
        std::vector<float> o = product(wo, att, E, qd, T);
        for (uint i = 0; i < T * E; i++) add(x.data(), o.data(), T * E, i);
        n = norm(x, ffn_norm, E, eps, T);
        std::vector<float> g = product(gate, n, F, E, T), u = product(up, n, F, E, T);
        for (uint i = 0; i < T * F; i++) silu_mul(g.data(), u.data(), T * F, i);
        std::vector<float> d = product(down, g, E, F, T);
        for (uint i = 0; i < T * E; i++) add(x.data(), d.data(), T * E, i);
    }
    std::vector<float> out_norm = read(E), head = read((size_t)V * E);
    std::fclose(f);
    std::vector<float> n = norm(x, out_norm, E, eps, T);
    std::vector<float> scores = product(head, n, V, E, T);

    FILE* o = std::fopen(argv[2], "wb");
    if (!o) { std::perror(argv[2]); return 1; }
    std::fwrite(scores.data(), 4, scores.size(), o);
    std::fclose(o);
    return 0;
}
