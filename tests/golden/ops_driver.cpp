// Calls the reference's own host functions for the per-layer operations (friday_cpu::rmsNorm, rope,
// decodeAttention, siluMul, addResidual: cpu_ops.h:12-28) at the sizes of the tests' tiny models and prints their
// outputs as JSON.  Links against the reference's libfriday_engine.a, built from its unmodified sources; see
// make_ops_golden.py.  Inputs come from a small generator that the Python side repeats, so only outputs are kept.
//   ops_driver > ops_golden.json
#include <cstdint>
#include <cstdio>
#include <vector>

#include "cpu_ops.h"

static uint32_t g_state = 1;
static float next_value(float scale) {                    // a linear congruential generator, values in [-scale, scale)
    g_state = (1103515245u * g_state + 12345u) & 0x7fffffffu;
    return ((float)g_state / 2147483648.0f * 2.0f - 1.0f) * scale;
}
static std::vector<float> draw(size_t n, float scale) {
    std::vector<float> v(n);
    for (auto& x : v) x = next_value(scale);
    return v;
}
static void print(const char* name, const std::vector<float>& v, bool last = false) {
    std::printf("  \"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) std::printf("%s%.9g", i ? ", " : "", v[i]);
    std::printf("]%s\n", last ? "" : ",");
}

struct Shape { const char* name; int width, heads, kv_heads, head_dim, inner; float theta, eps; };

int main() {
    const Shape shapes[2] = {{"A", 64, 4, 2, 16, 176, 10000.0f, 1e-6f}, {"B", 96, 3, 1, 32, 256, 1000000.0f, 1e-5f}};
    friday_cpu::ThreadPool pool(1);
    std::printf("{\n");
    for (int s = 0; s < 2; ++s) {
        const Shape& sh = shapes[s];
        g_state = 1000u + (uint32_t)s;
        char key[64];
        {   // rmsNorm
            std::vector<float> x = draw(sh.width, 3.0f), w = draw(sh.width, 1.0f), out(sh.width);
            friday_cpu::rmsNorm(x.data(), w.data(), out.data(), sh.width, sh.eps);
            std::snprintf(key, sizeof key, "%s.rms_norm", sh.name);
            print(key, out);
        }
        const int positions[4] = {0, 1, 63, 200};
        for (int p = 0; p < 4; ++p) {   // rope, NeoX pairing
            std::vector<float> q = draw((size_t)sh.heads * sh.head_dim, 1.0f), k = draw((size_t)sh.kv_heads * sh.head_dim, 1.0f);
            friday_cpu::rope(q.data(), k.data(), sh.head_dim, sh.heads, sh.kv_heads, positions[p], sh.theta, true, nullptr);
            q.insert(q.end(), k.begin(), k.end());
            std::snprintf(key, sizeof key, "%s.rope.%d", sh.name, positions[p]);
            print(key, q);
        }
        const int lengths[3] = {1, 37, 200};
        for (int l = 0; l < 3; ++l) {   // one query over `seq` keys
            const int seq = lengths[l], kv = sh.kv_heads * sh.head_dim;
            std::vector<float> q = draw((size_t)sh.heads * sh.head_dim, 2.0f), kc = draw((size_t)seq * kv, 1.0f),
                               vc = draw((size_t)seq * kv, 1.0f), out((size_t)sh.heads * sh.head_dim);
            friday_cpu::decodeAttention(q.data(), kc.data(), vc.data(), out.data(), seq, sh.heads, sh.kv_heads, sh.head_dim, pool);
            std::snprintf(key, sizeof key, "%s.attention.%d", sh.name, seq);
            print(key, out);
        }
        {   // siluMul and addResidual
            std::vector<float> gate = draw(sh.inner, 6.0f), up = draw(sh.inner, 2.0f);
            friday_cpu::siluMul(gate.data(), up.data(), sh.inner);
            std::snprintf(key, sizeof key, "%s.swiglu", sh.name);
            print(key, gate);
            std::vector<float> x = draw(sh.width, 2.0f), a = draw(sh.width, 2.0f);
            friday_cpu::addResidual(x.data(), a.data(), sh.width);
            std::snprintf(key, sizeof key, "%s.residual", sh.name);
            print(key, x, s == 1);
        }
    }
    std::printf("}\n");
    return 0;
}
