// A plain float32 Llama forward pass on the CPU in one C++ file: whole sequences, no cache, one
// function per part.  A second, independent statement of the formulas that tests/plain_llama.py
// states in Python (the two share nothing, not even a language), and the timed CPU baseline.
// The reference's float32 model is its CPU path, src/DotLLM.Models/Architectures/TransformerModel.cs:134-425.
//
//   llama_f32 MODEL.safetensors TOKENS.txt OUT.f32 key=value ...
//
// keys: layers hidden heads kv_heads head_dim intermediate vocab eps theta tied
//       scaling (0 none, 1 llama3) factor low high original
// TOKENS.txt holds the token ids of one sequence, whitespace separated.  OUT.f32 receives the logits
// [tokens, vocab] as little-endian float32.  Tensors are looked up by their HuggingFace names and
// must be stored as F32 (the tests write float32 folders for this program).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

struct Tensor {
    const float* data = nullptr;
    std::vector<long> shape;
};

static std::vector<char> g_file;
static std::map<std::string, Tensor> g_tensors;

[[noreturn]] static void die(const std::string& why) {
    std::fprintf(stderr, "llama_f32: %s\n", why.c_str());
    std::exit(2);
}

// The safetensors container: 8 bytes of header length, a JSON object name -> {dtype, shape,
// data_offsets}, then the data.  The header is scanned for exactly that shape of entry.
static void read_safetensors(const char* path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) die(std::string("cannot open ") + path);
    g_file.assign(std::istreambuf_iterator<char>(in), std::istreambuf_iterator<char>());
    if (g_file.size() < 8) die("file too short");
    uint64_t hlen = 0;
    std::memcpy(&hlen, g_file.data(), 8);
    if (8 + hlen > g_file.size()) die("header longer than the file");
    const std::string h(g_file.data() + 8, g_file.data() + 8 + hlen);
    const char* base = g_file.data() + 8 + hlen;
    size_t at = 0;
    while ((at = h.find("\"dtype\"", at)) != std::string::npos) {
        // the entry's name is the last quoted string before the '{' that opens this object
        const size_t open = h.rfind('{', at);
        const size_t q2 = h.rfind('"', open);
        const size_t q1 = h.rfind('"', q2 - 1);
        const std::string name = h.substr(q1 + 1, q2 - q1 - 1);
        const size_t close = h.find('}', at);
        const std::string body = h.substr(open, close - open);
        if (body.find("\"F32\"") == std::string::npos) die("tensor " + name + " is not stored as F32");
        Tensor t;
        size_t s = body.find("\"shape\"");
        s = body.find('[', s);
        size_t e = body.find(']', s);
        std::stringstream dims(body.substr(s + 1, e - s - 1));
        for (std::string d; std::getline(dims, d, ',');) t.shape.push_back(std::atol(d.c_str()));
        size_t o = body.find("\"data_offsets\"");
        o = body.find('[', o);
        const long begin = std::atol(body.c_str() + o + 1);
        t.data = reinterpret_cast<const float*>(base + begin);
        g_tensors[name] = t;
        at = close;
    }
}

static const float* weight(const std::string& name, long rows, long cols) {
    auto it = g_tensors.find(name);
    if (it == g_tensors.end()) die("missing tensor " + name);
    const auto& sh = it->second.shape;
    const bool ok = cols < 0 ? (sh.size() == 1 && sh[0] == rows) : (sh.size() == 2 && sh[0] == rows && sh[1] == cols);
    if (!ok) die("tensor " + name + " has another shape than the configuration gives");
    return it->second.data;
}

// y[t, o] = sum_i x[t, i] W[o, i]   (src/DotLLM.Cpu/Kernels/MatMul.cs:1121-1134, GemmF32: W is [out, in])
static std::vector<float> linear(const std::vector<float>& x, long T, long in, const float* W, long out) {
    std::vector<float> y((size_t)T * out);
    for (long t = 0; t < T; ++t)
        for (long o = 0; o < out; ++o) {
            const float* xr = &x[(size_t)t * in];
            const float* wr = W + (size_t)o * in;
            float acc = 0.f;
            for (long i = 0; i < in; ++i) acc += xr[i] * wr[i];
            y[(size_t)t * out + o] = acc;
        }
    return y;
}

// y_i = x_i * (1 / sqrt(sum x^2 / n + eps)) * w_i   (src/DotLLM.Cpu/Kernels/RmsNorm.cs:38-50)
static std::vector<float> rms_norm(const std::vector<float>& x, long T, long n, const float* w, float eps) {
    std::vector<float> y(x.size());
    for (long t = 0; t < T; ++t) {
        float ss = 0.f;
        for (long i = 0; i < n; ++i) ss += x[(size_t)t * n + i] * x[(size_t)t * n + i];
        const float inv = 1.0f / std::sqrt(ss / (float)n + eps);
        for (long i = 0; i < n; ++i) y[(size_t)t * n + i] = x[(size_t)t * n + i] * inv * w[i];
    }
    return y;
}

struct Scaling {
    int kind = 0;
    double factor = 1, low = 1, high = 4, original = 8192;
};

// f_i = theta^(-2i/d) (src/DotLLM.Cpu/Kernels/RoPE.cs:74); the llama3 rule rescales by wavelength:
// shorter than original/high: kept; longer than original/low: divided by factor; between: blended.
// (The reference applies no rescaling, src/DotLLM.Cpu/Kernels/RoPE.md:303.)
static std::vector<double> frequencies(long d, double theta, const Scaling& sc) {
    const double pi = 3.14159265358979323846;
    std::vector<double> f(d / 2);
    for (long i = 0; i < d / 2; ++i) {
        f[i] = 1.0 / std::pow(theta, (double)(2 * i) / (double)d);
        if (sc.kind == 1) {
            const double wavelen = 2.0 * pi / f[i];
            if (wavelen > sc.original / sc.low) {
                f[i] = f[i] / sc.factor;
            } else if (wavelen >= sc.original / sc.high) {
                const double s = (sc.original / wavelen - sc.low) / (sc.high - sc.low);
                f[i] = (1.0 - s) * f[i] / sc.factor + s * f[i];
            }
        }
    }
    return f;
}

// Half-split rotation of every head: (x[i], x[i + d/2]) -> (x0 c - x1 s, x0 s + x1 c)
// (src/DotLLM.Cpu/Kernels/RoPE.cs:250-256); tables in float64 rounded to float32 (:77-85).
static void rope(std::vector<float>& x, long T, long heads, long hd, const std::vector<double>& freq) {
    const long half = hd / 2;
    for (long t = 0; t < T; ++t)
        for (long i = 0; i < half; ++i) {
            const float c = (float)std::cos((double)t * freq[i]), s = (float)std::sin((double)t * freq[i]);
            for (long h = 0; h < heads; ++h) {
                float* p = &x[((size_t)t * heads + h) * hd];
                const float x0 = p[i], x1 = p[i + half];
                p[i] = x0 * c - x1 * s;
                p[i + half] = x0 * s + x1 * c;
            }
        }
}

// Scores, scale 1/sqrt(hd), causal mask, softmax with the maximum subtracted, weighted sum; query
// head h reads KV head h / (heads / kv_heads)   (src/DotLLM.Cpu/Kernels/Attention.cs:446-519, 47, 76, 106)
static std::vector<float> attention(const std::vector<float>& q, const std::vector<float>& k, const std::vector<float>& v, long T,
                                    long heads, long kv_heads, long hd) {
    std::vector<float> out((size_t)T * heads * hd);
    const float scale = 1.0f / std::sqrt((float)hd);
    const long group = heads / kv_heads;
    std::vector<float> w(T);
    for (long h = 0; h < heads; ++h) {
        const long kvh = h / group;
        for (long i = 0; i < T; ++i) {
            const float* qi = &q[((size_t)i * heads + h) * hd];
            float mx = -INFINITY;
            for (long j = 0; j <= i; ++j) {
                const float* kj = &k[((size_t)j * kv_heads + kvh) * hd];
                float dot = 0.f;
                for (long d = 0; d < hd; ++d) dot += qi[d] * kj[d];
                w[j] = dot * scale;
                mx = std::max(mx, w[j]);
            }
            float sum = 0.f;
            for (long j = 0; j <= i; ++j) {
                w[j] = std::exp(w[j] - mx);
                sum += w[j];
            }
            float* o = &out[((size_t)i * heads + h) * hd];
            for (long d = 0; d < hd; ++d) o[d] = 0.f;
            for (long j = 0; j <= i; ++j) {
                const float p = w[j] / sum;
                const float* vj = &v[((size_t)j * kv_heads + kvh) * hd];
                for (long d = 0; d < hd; ++d) o[d] += p * vj[d];
            }
        }
    }
    return out;
}

int main(int argc, char** argv) {
    if (argc < 4) die("usage: llama_f32 MODEL.safetensors TOKENS.txt OUT.f32 key=value ...");
    std::map<std::string, double> c;
    for (int i = 4; i < argc; ++i) {
        const char* eq = std::strchr(argv[i], '=');
        if (!eq) die(std::string("not key=value: ") + argv[i]);
        c[std::string(argv[i], (size_t)(eq - argv[i]))] = std::atof(eq + 1);
    }
    for (const char* key : {"layers", "hidden", "heads", "kv_heads", "head_dim", "intermediate", "vocab", "eps", "theta", "tied"})
        if (!c.count(key)) die(std::string("missing ") + key);
    const long L = (long)c["layers"], H = (long)c["hidden"], nh = (long)c["heads"], nkv = (long)c["kv_heads"], hd = (long)c["head_dim"],
               I = (long)c["intermediate"], V = (long)c["vocab"];
    const float eps = (float)c["eps"];
    Scaling sc;
    sc.kind = (int)c["scaling"];
    if (sc.kind == 1) sc.factor = c["factor"], sc.low = c["low"], sc.high = c["high"], sc.original = c["original"];
    read_safetensors(argv[1]);
    std::vector<long> tokens;
    {
        std::ifstream in(argv[2]);
        for (long t; in >> t;) tokens.push_back(t);
    }
    const long T = (long)tokens.size();
    if (T == 0) die("no tokens");
    const auto t0 = std::chrono::steady_clock::now();

    // h[t] = E[token[t]], no scale (TransformerModel.cs:729-749)
    const float* E = weight("model.embed_tokens.weight", V, H);
    std::vector<float> h((size_t)T * H);
    for (long t = 0; t < T; ++t) {
        if (tokens[t] < 0 || tokens[t] >= V) die("token id outside the vocabulary");
        std::memcpy(&h[(size_t)t * H], E + (size_t)tokens[t] * H, sizeof(float) * H);
    }
    const std::vector<double> freq = frequencies(hd, c["theta"], sc);
    // r = h; h = r + attn(norm(h)); r = h; h = r + ffn(norm(h))   (TransformerModel.cs:185-392)
    for (long l = 0; l < L; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        std::vector<float> n = rms_norm(h, T, H, weight(p + "input_layernorm.weight", H, -1), eps);
        std::vector<float> q = linear(n, T, H, weight(p + "self_attn.q_proj.weight", nh * hd, H), nh * hd);
        std::vector<float> k = linear(n, T, H, weight(p + "self_attn.k_proj.weight", nkv * hd, H), nkv * hd);
        std::vector<float> v = linear(n, T, H, weight(p + "self_attn.v_proj.weight", nkv * hd, H), nkv * hd);
        rope(q, T, nh, hd, freq);
        rope(k, T, nkv, hd, freq);
        std::vector<float> a = attention(q, k, v, T, nh, nkv, hd);
        std::vector<float> o = linear(a, T, nh * hd, weight(p + "self_attn.o_proj.weight", H, nh * hd), H);
        for (size_t i = 0; i < h.size(); ++i) h[i] += o[i];
        n = rms_norm(h, T, H, weight(p + "post_attention_layernorm.weight", H, -1), eps);
        std::vector<float> g = linear(n, T, H, weight(p + "mlp.gate_proj.weight", I, H), I);
        std::vector<float> u = linear(n, T, H, weight(p + "mlp.up_proj.weight", I, H), I);
        // silu(g) * u with sigmoid = 1 / (1 + exp(-g))   (src/DotLLM.Cpu/Kernels/FusedOps.cs:69-78)
        for (size_t i = 0; i < g.size(); ++i) g[i] = g[i] * (1.0f / (1.0f + std::exp(-g[i]))) * u[i];
        std::vector<float> d = linear(g, T, I, weight(p + "mlp.down_proj.weight", H, I), H);
        for (size_t i = 0; i < h.size(); ++i) h[i] += d[i];
    }
    std::vector<float> n = rms_norm(h, T, H, weight("model.norm.weight", H, -1), eps);
    // no output matrix: the embedding table (src/DotLLM.Models/Architectures/TransformerWeights.cs:205-220)
    const float* head = c["tied"] != 0 ? E : weight("lm_head.weight", V, H);
    std::vector<float> logits = linear(n, T, H, head, V);
    const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::ofstream out(argv[3], std::ios::binary);
    out.write(reinterpret_cast<const char*>(logits.data()), (std::streamsize)(logits.size() * sizeof(float)));
    std::printf("{\"tokens\": %ld, \"seconds\": %.6f, \"tokens_per_second\": %.1f}\n", T, seconds, (double)T / seconds);
    return 0;
}
