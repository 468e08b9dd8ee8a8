// The plain C++ twin of the kernels: every part of the Llama dense decoder as a short loop
// on the host, one function a part, and the whole model as their sequence.  It is what each
// CUDA kernel of this library is held against beside the NumPy oracle of the tests, and it is
// the timed CPU baseline of the tiny workloads.  Whole sequences, no cache, no batching, no
// vector intrinsics: float values, double sums.
//
// The formulas are the reference's (Harshil089/Borrowed-Compute), cited by the file's path in
// that project:
//   embedding                 crates/bc-infer/src/model.rs:270-280
//   RMSNorm                   crates/bc-infer/src/model.rs:381-389; gpu/kernels.h:226-233
//   products                  crates/bc-infer/src/quant.rs:365-372 (out[i][r] = sum_c W[r][c] x[i][c])
//   rotary encoding           crates/bc-infer/src/model.rs:391-403; gpu/kernels.h:237-248
//   attention                 crates/bc-infer/src/model.rs:448-481
//   SwiGLU                    crates/bc-infer/src/model.rs:341-345; gpu/kernels.h:330
//   layer and model order     crates/bc-infer/src/model.rs:320-346, 361-370; lib.rs:50-54
//   sampling                  crates/bc-infer/src/sample.rs:24-71
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

extern "C" {

// out[r, :] = table[tokens[r], :]; -1 if a token lies outside the table.
int twin_embed(const float* table, int vocab, int width, const int* tokens, int rows, float* out) {
    for (int r = 0; r < rows; r++) {
        if (tokens[r] < 0 || tokens[r] >= vocab) return -1;
        std::memcpy(out + (size_t)r * width, table + (size_t)tokens[r] * width, sizeof(float) * width);
    }
    return 0;
}

// out = x * (1 / sqrt(mean(x^2) + eps)) * w, row by row: eps inside the root, the weight after the scale.
void twin_rmsnorm(const float* x, const float* w, float* out, int rows, int width, float eps) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * width;
        double ss = 0.0;
        for (int c = 0; c < width; c++) ss += (double)xr[c] * xr[c];
        const double scale = 1.0 / std::sqrt(ss / width + (double)eps);
        for (int c = 0; c < width; c++) out[(size_t)r * width + c] = (float)(xr[c] * scale * w[c]);
    }
}

// out[i, n] = sum_k x[i, k] * w[n, k]  (weights are [out, in], as stored).
void twin_linear(const float* x, const float* w, float* out, int rows, int n_out, int k_in) {
    for (int i = 0; i < rows; i++)
        for (int n = 0; n < n_out; n++) {
            double s = 0.0;
            const float* xi = x + (size_t)i * k_in;
            const float* wn = w + (size_t)n * k_in;
            for (int k = 0; k < k_in; k++) s += (double)xi[k] * wn[k];
            out[(size_t)i * n_out + n] = (float)s;
        }
}

// One frequency per rotated pair: theta^(-2i/d), slowed by the llama3 rule if `factor` > 0
// (wavelengths shorter than original / high keep their frequency, longer than original / low
// are divided by `factor`, those between blend the two linearly in original / wavelength);
// computed in double, rounded to float once.  The reference divides by stored per-pair
// factors (crates/bc-infer/src/model.rs:208-211); this rule is what produces them.
void twin_inv_freq(int d, double theta, double factor, double low, double high, double original, float* out) {
    const double pi = 3.14159265358979323846;
    for (int i = 0; i < d / 2; i++) {
        double f = std::pow(theta, -2.0 * i / d);
        if (factor > 0.0) {
            const double wavelen = 2.0 * pi / f;
            if (wavelen > original / low) f = f / factor;
            else if (wavelen >= original / high) {
                const double t = (original / wavelen - low) / (high - low);
                f = (1.0 - t) * f / factor + t * f;
            }
        }
        out[i] = (float)f;
    }
}

// Rotates every head of x [rows, heads, d] in place by positions[r] * inv_freq[i]; the angle is
// the float product of the two, as in the reference.  pairing 0: (i, i + d/2); 1: (2i, 2i + 1).
void twin_rope(float* x, const int* positions, int rows, int heads, int d, const float* inv_freq, int pairing) {
    const int half = d / 2;
    for (int r = 0; r < rows; r++)
        for (int i = 0; i < half; i++) {
            const float angle = (float)positions[r] * inv_freq[i];
            const double c = std::cos((double)angle), s = std::sin((double)angle);
            const int a = pairing ? 2 * i : i, b = pairing ? 2 * i + 1 : i + half;
            for (int h = 0; h < heads; h++) {
                float* v = x + ((size_t)r * heads + h) * d;
                const double x0 = v[a], x1 = v[b];
                v[a] = (float)(x0 * c - x1 * s);
                v[b] = (float)(x0 * s + x1 * c);
            }
        }
}

// Causal grouped-query attention over one whole sequence: q [rows, heads, d], k and v
// [rows, kv_heads, d]; row i sees rows max(0, i - window + 1) .. i (all of 0 .. i if window is 0).
void twin_attention(const float* q, const float* k, const float* v, float* out, int rows, int heads, int kv_heads, int d, int window) {
    const int group = heads / kv_heads;
    const double scale = 1.0 / std::sqrt((double)d);
    std::vector<double> p(rows);
    for (int i = 0; i < rows; i++)
        for (int h = 0; h < heads; h++) {
            const int g = h / group, lo = window > 0 && i + 1 > window ? i + 1 - window : 0;
            const float* qi = q + ((size_t)i * heads + h) * d;
            double top = -INFINITY;
            for (int t = lo; t <= i; t++) {
                const float* kt = k + ((size_t)t * kv_heads + g) * d;
                double s = 0.0;
                for (int c = 0; c < d; c++) s += (double)qi[c] * kt[c];
                p[t] = s * scale;
                top = std::max(top, p[t]);
            }
            double sum = 0.0;
            for (int t = lo; t <= i; t++) sum += (p[t] = std::exp(p[t] - top));
            for (int c = 0; c < d; c++) {
                double acc = 0.0;
                for (int t = lo; t <= i; t++) acc += p[t] * v[((size_t)t * kv_heads + g) * d + c];
                out[((size_t)i * heads + h) * d + c] = (float)(acc / sum);
            }
        }
}

// out = g / (1 + e^-g) * u, element by element.
void twin_swiglu(const float* gate, const float* up, float* out, long long n) {
    for (long long i = 0; i < n; i++) out[i] = (float)((double)gate[i] / (1.0 + std::exp(-(double)gate[i])) * up[i]);
}

// The first largest score wins.
int twin_argmax(const float* scores, int n) {
    int best = 0;
    for (int i = 1; i < n; i++)
        if (scores[i] > scores[best]) best = i;
    return best;
}

static double twin_uniform(uint64_t seed) {
    uint64_t z = seed + 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    return (double)(z >> 40) / 16777216.0;
}

// One draw: greedy at temperature <= 0; else weights e^((s - max)/T), sorted descending (ties by
// ascending id), cut to the shortest prefix whose share reaches top_p, and a uniform number from
// seed ^ step * golden ratio walked down the kept list.
int twin_sample(const float* scores, int n, float temperature, float top_p, uint64_t seed, uint64_t step) {
    if (!(temperature > 0.0f)) return twin_argmax(scores, n);
    const double top = scores[twin_argmax(scores, n)];
    std::vector<double> w(n);
    double total = 0.0;
    for (int i = 0; i < n; i++) total += (w[i] = std::exp(((double)scores[i] - top) / temperature));
    std::vector<int> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return w[a] > w[b]; });
    int keep = 0;
    double mass = 0.0, kept = 0.0;
    for (int i : order) {
        keep++;
        mass += w[i] / total;
        kept += w[i];
        if (mass >= top_p) break;
    }
    double r = twin_uniform(seed ^ (step * 0x9e3779b97f4a7c15ull)) * kept;
    for (int j = 0; j < keep; j++) {
        r -= w[order[j]];
        if (r <= 0.0) return order[j];
    }
    return order[0];
}

// One model's sizes and tensors, [out, in] matrices as stored.  Per-layer tensors are arrays
// of `layers` pointers.  `head` may equal `embed` (a tied head).
struct TwinModel {
    int layers, hidden, heads, kv_heads, head_dim, intermediate, vocab, pairing;
    float eps;
    const float* inv_freq;   // [head_dim / 2]
    const float* embed;      // [vocab, hidden]
    const float* const* ln1; // [hidden]
    const float* const* wq;  // [heads * head_dim, hidden]
    const float* const* wk;  // [kv_heads * head_dim, hidden]
    const float* const* wv;
    const float* const* wo;  // [hidden, heads * head_dim]
    const float* const* ln2;
    const float* const* gate;  // [intermediate, hidden]
    const float* const* up;
    const float* const* down;  // [hidden, intermediate]
    const float* norm;
    const float* head;       // [vocab, hidden]
};

// Scores after every token of one sequence fed from position 0: out [n, vocab].  -1 on a bad token.
int twin_logits(const TwinModel* m, const int* tokens, int n, float* out) {
    const int E = m->hidden, H = m->heads, G = m->kv_heads, D = m->head_dim, F = m->intermediate;
    std::vector<float> x((size_t)n * E), h((size_t)n * E), q((size_t)n * H * D), k((size_t)n * G * D), v((size_t)n * G * D),
        att((size_t)n * H * D), proj((size_t)n * E), g((size_t)n * F), u((size_t)n * F);
    std::vector<int> pos(n);
    std::iota(pos.begin(), pos.end(), 0);
    if (twin_embed(m->embed, m->vocab, E, tokens, n, x.data()) != 0) return -1;
    for (int l = 0; l < m->layers; l++) {
        twin_rmsnorm(x.data(), m->ln1[l], h.data(), n, E, m->eps);
        twin_linear(h.data(), m->wq[l], q.data(), n, H * D, E);
        twin_linear(h.data(), m->wk[l], k.data(), n, G * D, E);
        twin_linear(h.data(), m->wv[l], v.data(), n, G * D, E);
        twin_rope(q.data(), pos.data(), n, H, D, m->inv_freq, m->pairing);
        twin_rope(k.data(), pos.data(), n, G, D, m->inv_freq, m->pairing);
        twin_attention(q.data(), k.data(), v.data(), att.data(), n, H, G, D, 0);
        twin_linear(att.data(), m->wo[l], proj.data(), n, E, H * D);
        for (size_t i = 0; i < x.size(); i++) x[i] += proj[i];
        twin_rmsnorm(x.data(), m->ln2[l], h.data(), n, E, m->eps);
        twin_linear(h.data(), m->gate[l], g.data(), n, F, E);
        twin_linear(h.data(), m->up[l], u.data(), n, F, E);
        twin_swiglu(g.data(), u.data(), g.data(), (long long)n * F);
        twin_linear(g.data(), m->down[l], proj.data(), n, E, F);
        for (size_t i = 0; i < x.size(); i++) x[i] += proj[i];
    }
    twin_rmsnorm(x.data(), m->norm, h.data(), n, E, m->eps);
    twin_linear(h.data(), m->head, out, n, m->vocab, E);
    return 0;
}

// Continues one prompt by recomputing the whole sequence every step; a stop id ends the text
// and is not part of it.  Returns how many ids were written to `out`, or -1 on a bad token.
int twin_generate(const TwinModel* m, const int* prompt, int n_prompt, int max_tokens, float temperature, float top_p, uint64_t seed,
                  const int* stops, int n_stops, int* out) {
    std::vector<int> seq(prompt, prompt + n_prompt);
    std::vector<float> scores;
    int made = 0;
    while (made < max_tokens) {
        scores.resize((size_t)seq.size() * m->vocab);
        if (twin_logits(m, seq.data(), (int)seq.size(), scores.data()) != 0) return -1;
        const float* row = scores.data() + (seq.size() - 1) * (size_t)m->vocab;
        const int tok = twin_sample(row, m->vocab, temperature, top_p, seed, (uint64_t)(seq.size() - 1));
        if (std::find(stops, stops + n_stops, tok) != stops + n_stops) break;
        out[made++] = tok;
        seq.push_back(tok);
    }
    return made;
}

}  // extern "C"
