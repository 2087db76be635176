// A scalar restatement of the dense decoder, token by token, with sequential float32 accumulation:
// what a single-sequence CPU decoder of this architecture computes, written from the formulas the
// plain implementation cites (embedding row, RMSNorm with eps inside the square root, q/k/v
// projections with optional biases, rotary encoding from a table built in float32, a cache of all
// earlier keys and values, attention with scale 1/sqrt(head_dim) applied to the finished dot product
// and a max-subtracted softmax, output projection, SwiGLU, final norm, head).  It is an independent
// anchor for tests/plain_impl.py: another language, loops instead of tensor expressions, a cache
// instead of whole-sequence attention.  Not part of the product; the GPU code never sees it.
//
//   scalar_decoder <weights.bin> <tokens.txt> <logits.bin> hidden layers heads kv_heads head_dim inter
//                  vocab rope_theta eps bias tied style
//
// weights.bin: float32, in the order read below.  logits.bin: float32 [n_tokens, vocab].
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

typedef std::vector<float> vec;

static vec read_floats(FILE* f, size_t n) {
    vec v(n);
    if (fread(v.data(), sizeof(float), n, f) != n) { fprintf(stderr, "weights file too short\n"); exit(2); }
    return v;
}

// y[r] = sum_c W[r, c] x[c] (+ b[r]), row-major W, accumulated left to right in float32
static void matvec(const vec& W, const vec* b, const float* x, float* y, int rows, int cols) {
    for (int r = 0; r < rows; ++r) {
        float acc = 0.f;
        const float* w = &W[(size_t)r * cols];
        for (int c = 0; c < cols; ++c) acc += w[c] * x[c];
        y[r] = b ? acc + (*b)[r] : acc;
    }
}

static void rmsnorm(const float* x, const vec& w, float eps, float* y, int n) {
    float ss = 0.f;
    for (int i = 0; i < n; ++i) ss += x[i] * x[i];
    const float scale = 1.0f / std::sqrt(ss / (float)n + eps);
    for (int i = 0; i < n; ++i) y[i] = x[i] * scale * w[i];
}

struct Layer {
    vec attn_norm, wq, wk, wv, bq, bk, bv, wo, ffn_norm, wg, wu, wd;
};

int main(int argc, char** argv) {
    if (argc != 16) { fprintf(stderr, "usage: see the header of scalar_decoder.cpp\n"); return 2; }
    const int H = atoi(argv[4]), L = atoi(argv[5]), nh = atoi(argv[6]), nkv = atoi(argv[7]), hd = atoi(argv[8]);
    const int I = atoi(argv[9]), V = atoi(argv[10]);
    const float theta = (float)atof(argv[11]), eps = (float)atof(argv[12]);
    const int bias = atoi(argv[13]), tied = atoi(argv[14]), style = atoi(argv[15]);   // style 0: pairs (i, i + hd/2); 1: (2i, 2i+1)
    const int qd = nh * hd, kvd = nkv * hd, half = hd / 2, n_rep = nh / nkv;

    FILE* f = fopen(argv[1], "rb");
    if (!f) { perror(argv[1]); return 2; }
    vec embed = read_floats(f, (size_t)V * H);
    std::vector<Layer> layers(L);
    for (Layer& l : layers) {
        l.attn_norm = read_floats(f, H);
        l.wq = read_floats(f, (size_t)qd * H);
        l.wk = read_floats(f, (size_t)kvd * H);
        l.wv = read_floats(f, (size_t)kvd * H);
        if (bias) { l.bq = read_floats(f, qd); l.bk = read_floats(f, kvd); l.bv = read_floats(f, kvd); }
        l.wo = read_floats(f, (size_t)H * qd);
        l.ffn_norm = read_floats(f, H);
        l.wg = read_floats(f, (size_t)I * H);
        l.wu = read_floats(f, (size_t)I * H);
        l.wd = read_floats(f, (size_t)H * I);
    }
    vec final_norm = read_floats(f, H);
    vec head = tied ? embed : read_floats(f, (size_t)V * H);
    fclose(f);

    std::vector<int> tokens;
    f = fopen(argv[2], "r");
    if (!f) { perror(argv[2]); return 2; }
    for (int t; fscanf(f, "%d", &t) == 1;) tokens.push_back(t);
    fclose(f);
    const int n = (int)tokens.size();

    // angle tables: exponent = 2i / hd, theta_i = 1 / base^exponent, angle = pos * theta_i, all in float32
    vec cos_t((size_t)n * half), sin_t((size_t)n * half);
    for (int pos = 0; pos < n; ++pos)
        for (int i = 0; i < half; ++i) {
            const float exponent = (float)(2 * i) / (float)hd;
            const float th = 1.0f / std::pow(theta, exponent);
            const float angle = (float)pos * th;
            cos_t[(size_t)pos * half + i] = (float)std::cos((double)angle);
            sin_t[(size_t)pos * half + i] = (float)std::sin((double)angle);
        }

    std::vector<vec> kcache(L, vec((size_t)n * kvd)), vcache(L, vec((size_t)n * kvd));
    vec h(H), xn(H), q(qd), k(kvd), v(kvd), mixed(qd), proj(H), g(I), u(I), scores(n), logits(V);
    FILE* out = fopen(argv[3], "wb");
    if (!out) { perror(argv[3]); return 2; }
    const float scale = 1.0f / std::sqrt((float)hd);

    for (int pos = 0; pos < n; ++pos) {
        for (int i = 0; i < H; ++i) h[i] = embed[(size_t)tokens[pos] * H + i];
        for (int li = 0; li < L; ++li) {
            const Layer& l = layers[li];
            rmsnorm(h.data(), l.attn_norm, eps, xn.data(), H);
            matvec(l.wq, bias ? &l.bq : nullptr, xn.data(), q.data(), qd, H);
            matvec(l.wk, bias ? &l.bk : nullptr, xn.data(), k.data(), kvd, H);
            matvec(l.wv, bias ? &l.bv : nullptr, xn.data(), v.data(), kvd, H);
            // rotate every q head and every k head by the position's angles
            for (int hh = 0; hh < nh + nkv; ++hh) {
                float* x = hh < nh ? &q[(size_t)hh * hd] : &k[(size_t)(hh - nh) * hd];
                for (int i = 0; i < half; ++i) {
                    const int i0 = style == 0 ? i : 2 * i, i1 = style == 0 ? i + half : 2 * i + 1;
                    const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
                    const float x0 = x[i0], x1 = x[i1];
                    x[i0] = x0 * c - x1 * s;
                    x[i1] = x0 * s + x1 * c;
                }
            }
            for (int i = 0; i < kvd; ++i) {
                kcache[li][(size_t)pos * kvd + i] = k[i];
                vcache[li][(size_t)pos * kvd + i] = v[i];
            }
            // attention of head hh over the cached positions 0..pos of its kv head
            for (int hh = 0; hh < nh; ++hh) {
                const int kvh = hh / n_rep;
                float m = -INFINITY;
                for (int j = 0; j <= pos; ++j) {
                    float dot = 0.f;
                    for (int d = 0; d < hd; ++d) dot += q[(size_t)hh * hd + d] * kcache[li][(size_t)j * kvd + kvh * hd + d];
                    scores[j] = dot * scale;
                    if (scores[j] > m) m = scores[j];
                }
                float z = 0.f;
                for (int j = 0; j <= pos; ++j) { scores[j] = std::exp(scores[j] - m); z += scores[j]; }
                const float inv = 1.0f / z;
                for (int d = 0; d < hd; ++d) {
                    float acc = 0.f;
                    for (int j = 0; j <= pos; ++j) acc += scores[j] * inv * vcache[li][(size_t)j * kvd + kvh * hd + d];
                    mixed[(size_t)hh * hd + d] = acc;
                }
            }
            matvec(l.wo, nullptr, mixed.data(), proj.data(), H, qd);
            for (int i = 0; i < H; ++i) h[i] += proj[i];
            rmsnorm(h.data(), l.ffn_norm, eps, xn.data(), H);
            matvec(l.wg, nullptr, xn.data(), g.data(), I, H);
            matvec(l.wu, nullptr, xn.data(), u.data(), I, H);
            for (int i = 0; i < I; ++i) {
                const float x = g[i];
                const float silu = x >= 0.f ? x / (1.0f + std::exp(-x)) : x * std::exp(x) / (1.0f + std::exp(x));
                g[i] = silu * u[i];
            }
            matvec(l.wd, nullptr, g.data(), proj.data(), H, I);
            for (int i = 0; i < H; ++i) h[i] += proj[i];
        }
        rmsnorm(h.data(), final_norm, eps, xn.data(), H);
        matvec(head, nullptr, xn.data(), logits.data(), V, H);
        fwrite(logits.data(), sizeof(float), V, out);
    }
    fclose(out);
    return 0;
}
