// A second plain restatement of the Mistral dense decoder, for tests and for a timed CPU
// baseline.  Where tests/plain/mistral_plain.py runs whole sequences with matrix products and
// no cache, this one runs the way rglonek/torchless-rs runs: one token of one sequence per
// forward pass, keys and values kept in a cache [layer][kv head][position][head_dim], every
// output a sequential 32-bit dot product (src/model/mod.rs:430-447, src/loader/parameters.rs:551-594).
// The two share no code and no structure; tests require them to agree before either is used
// to check the engine.  Nothing here was checked against a run of the reference (no Rust toolchain
// where this is built): it rests on the cited formulas.
//
//   mistral_plain_onetoken <model_dir> <tokens.txt> <logits.f32>     logits [n, vocab] of one sequence
//   mistral_plain_onetoken --time-layer <config.json> <context> <repeats>
//       times one layer's single-token forward (random weights) and the head; prints JSON
//
// Reads config.json and model.safetensors (F32, BF16, F16) with a scanner that is just enough
// for those two files.  Plain C++17, one thread, no library beyond the standard one.
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

using std::string;
using std::vector;

static void die(const string& msg) { fprintf(stderr, "mistral_plain_onetoken: %s\n", msg.c_str()); exit(2); }

static string read_file(const string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) die("cannot open " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

// ---- just enough JSON: the value text that follows "key": at the top level of `text` ----------
static bool find_value(const string& text, const string& key, string* out) {
  const string pat = "\"" + key + "\"";
  size_t at = 0;
  while ((at = text.find(pat, at)) != string::npos) {
    size_t p = at + pat.size();
    while (p < text.size() && isspace((unsigned char)text[p])) ++p;
    if (p < text.size() && text[p] == ':') {
      ++p;
      while (p < text.size() && isspace((unsigned char)text[p])) ++p;
      size_t q = p;
      int depth = 0;
      bool in_str = false;
      for (; q < text.size(); ++q) {
        const char c = text[q];
        if (in_str) { if (c == '\\') ++q; else if (c == '"') in_str = false; continue; }
        if (c == '"') in_str = true;
        else if (c == '[' || c == '{') ++depth;
        else if (c == ']' || c == '}') { if (depth == 0) break; --depth; }
        else if (c == ',' && depth == 0) break;
      }
      *out = text.substr(p, q - p);
      while (!out->empty() && isspace((unsigned char)out->back())) out->pop_back();
      return true;
    }
    at += pat.size();
  }
  return false;
}
static double num_or(const string& text, const string& key, double dflt, bool* found = nullptr) {
  string v;
  const bool ok = find_value(text, key, &v) && v != "null";
  if (found) *found = ok;
  return ok ? atof(v.c_str()) : dflt;
}

// ---- configuration: the keys and defaults of src/loader/formats/safetensors.rs:701-765 ----------
struct Config {
  int hidden, inter, layers, heads, kv_heads, head_dim, vocab, window;   // window 0 = none
  float theta, eps;
};
static Config read_config(const string& text) {
  Config c;
  bool ok;
  c.hidden = (int)num_or(text, "hidden_size", 0, &ok); if (!ok) die("config.json: hidden_size is missing");
  c.inter = (int)num_or(text, "intermediate_size", 0, &ok); if (!ok) die("config.json: intermediate_size is missing");
  c.layers = (int)num_or(text, "num_hidden_layers", 0, &ok); if (!ok) die("config.json: num_hidden_layers is missing");
  c.heads = (int)num_or(text, "num_attention_heads", 0, &ok); if (!ok) die("config.json: num_attention_heads is missing");
  c.vocab = (int)num_or(text, "vocab_size", 0, &ok); if (!ok) die("config.json: vocab_size is missing");
  c.kv_heads = (int)num_or(text, "num_key_value_heads", c.heads);        // default = heads (:731-735)
  c.head_dim = (int)num_or(text, "head_dim", c.hidden / c.heads);        // src/model/mod.rs:143
  c.theta = (float)num_or(text, "rope_theta", 10000.0);                  // gguf.rs:1200
  c.eps = (float)num_or(text, "rms_norm_eps", 1e-5);                     // gguf.rs:1202
  c.window = (int)num_or(text, "sliding_window", 0);
  return c;
}

// ---- safetensors: 8-byte header length, JSON header, data (src/loader/formats/safetensors.rs:196-356) ----
static float bf16_to_f32(uint16_t h) {   // bits << 16 (src/loader/parameters.rs:573-580)
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 31, man = h & 1023;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {   // subnormal: renormalise
      int e = -1;
      uint32_t m = man;
      do { ++e; m <<= 1; } while ((m & 1024) == 0);
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 1023) << 13);
    }
  } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
  else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
struct Weights {
  string blob, header;
  size_t data0 = 0;
  explicit Weights(const string& path) : blob(read_file(path)) {
    if (blob.size() < 8) die("model.safetensors: file too small");
    uint64_t n;
    memcpy(&n, blob.data(), 8);
    if (8 + n > blob.size()) die("model.safetensors: invalid header size");
    header = blob.substr(8, n);
    data0 = 8 + n;
  }
  vector<float> get(const string& name, size_t expect) const {
    string obj, dt, offs;
    if (!find_value(header, name, &obj)) die("Tensor '" + name + "' not found");
    if (!find_value(obj, "dtype", &dt) || !find_value(obj, "data_offsets", &offs)) die("bad entry for " + name);
    size_t a = 0, b = 0;
    if (sscanf(offs.c_str(), "[%zu,%zu]", &a, &b) != 2 && sscanf(offs.c_str(), "[%zu, %zu]", &a, &b) != 2)
      die("bad data_offsets for " + name);
    if (data0 + b > blob.size()) die("data of " + name + " exceeds the file");
    const char* p = blob.data() + data0 + a;
    vector<float> out(expect);
    if (dt == "\"F32\"") {
      if (b - a != expect * 4) die("wrong size of " + name);
      memcpy(out.data(), p, expect * 4);
    } else if (dt == "\"BF16\"" || dt == "\"F16\"") {
      if (b - a != expect * 2) die("wrong size of " + name);
      for (size_t i = 0; i < expect; ++i) {
        uint16_t h;
        memcpy(&h, p + 2 * i, 2);
        out[i] = dt == "\"BF16\"" ? bf16_to_f32(h) : f16_to_f32(h);
      }
    } else die("Unsupported dtype " + dt + " of " + name);
    return out;
  }
};

// ---- the parts, one function each ------------------------------------------------------------
// y[o] = sum_i W[o, i] x[i], one sequential 32-bit accumulation per output
// (src/loader/parameters.rs:551-594).
static void matvec(const float* w, const float* x, float* y, int out, int in) {
  for (int o = 0; o < out; ++o) {
    const float* row = w + (size_t)o * in;
    float acc = 0.0f;
    for (int i = 0; i < in; ++i) acc += row[i] * x[i];
    y[o] = acc;
  }
}
// y = x / sqrt(mean(x^2) + eps) * w: divide, then multiply (src/kernels/mod.rs:558-568).
static void rmsnorm(const float* x, const float* w, float eps, float* y, int n) {
  float ss = 0.0f;
  for (int i = 0; i < n; ++i) ss += x[i] * x[i];
  const float rms = sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; ++i) y[i] = (x[i] / rms) * w[i];
}
// Half-split rotation of one head at position pos (src/kernels/mod.rs:572-608).
static void rope(float* x, int hd, const float* inv_freq, int pos) {
  const int half = hd / 2;
  for (int i = 0; i < half; ++i) {
    const float ang = inv_freq[i] * (float)pos;
    const float c = cosf(ang), s = sinf(ang);
    const float a = x[i], b = x[i + half];
    x[i] = a * c - b * s;
    x[i + half] = a * s + b * c;
  }
}
static float silu(float z) { return z / (1.0f + expf(-z)); }   // src/kernels/mod.rs:546-548

struct Layer {
  vector<float> n1, n2, wq, wk, wv, wo, wg, wu, wd;
};
struct Model {
  Config c;
  vector<float> embed, norm, head, inv_freq;
  vector<Layer> layers;
  vector<float> kc, vc;   // [layer][kv head][position][head_dim] (src/model/kv_cache.rs:23-53)
  int cap = 0;
  void alloc_cache(int max_pos) {
    cap = max_pos;
    kc.assign((size_t)c.layers * c.kv_heads * cap * c.head_dim, 0.0f);
    vc = kc;
  }
  float* kat(int l, int h, int p) { return kc.data() + (((size_t)l * c.kv_heads + h) * cap + p) * c.head_dim; }
  float* vat(int l, int h, int p) { return vc.data() + (((size_t)l * c.kv_heads + h) * cap + p) * c.head_dim; }

  // One token at position pos; h is the residual stream [hidden], updated in place.
  // Pre-norm block: h += Attn(Norm1(h)); h += MLP(Norm2(h)) (src/model/modules/layer.rs:28-56).
  void layer_forward(int l, float* h, int pos) {
    const Layer& L = layers[l];
    const int H = c.hidden, nh = c.heads, nkv = c.kv_heads, hd = c.head_dim, I = c.inter;
    vector<float> xn(H), q(nh * hd), k(nkv * hd), v(nkv * hd), ctx(nh * hd, 0.0f), out(H), scores(pos + 1);
    rmsnorm(h, L.n1.data(), c.eps, xn.data(), H);
    matvec(L.wq.data(), xn.data(), q.data(), nh * hd, H);      // src/model/modules/attention.rs:46-53
    matvec(L.wk.data(), xn.data(), k.data(), nkv * hd, H);
    matvec(L.wv.data(), xn.data(), v.data(), nkv * hd, H);
    for (int i = 0; i < nh; ++i) rope(q.data() + i * hd, hd, inv_freq.data(), pos);   // :69-72
    for (int i = 0; i < nkv; ++i) rope(k.data() + i * hd, hd, inv_freq.data(), pos);
    for (int i = 0; i < nkv; ++i) {                                                   // rotate, then cache: :75
      memcpy(kat(l, i, pos), k.data() + i * hd, hd * sizeof(float));
      memcpy(vat(l, i, pos), v.data() + i * hd, hd * sizeof(float));
    }
    const int group = nh / nkv;
    const float scale = 1.0f / sqrtf((float)hd);                                     // :83
    // keys 0..pos (:90); with a window W only keys pos-W+1..pos (the inequality of
    // src/model/models/gpt_oss.rs:168-176, which the reference's Mistral does not apply)
    const int lo = c.window > 0 && pos - c.window + 1 > 0 ? pos - c.window + 1 : 0;
    for (int hq = 0; hq < nh; ++hq) {
      const int kvh = hq / group;
      const float* qh = q.data() + hq * hd;
      float mx = -INFINITY;
      for (int i = lo; i <= pos; ++i) {                                               // src/kernels/mod.rs:511-526
        const float* kr = kat(l, kvh, i);
        float acc = 0.0f;
        for (int d = 0; d < hd; ++d) acc += kr[d] * qh[d];
        scores[i] = acc * scale;
        if (scores[i] > mx) mx = scores[i];
      }
      float sum = 0.0f;                                                               // src/kernels/mod.rs:538-543
      for (int i = lo; i <= pos; ++i) { scores[i] = expf(scores[i] - mx); sum += scores[i]; }
      for (int i = lo; i <= pos; ++i) scores[i] = scores[i] / sum;
      float* ch = ctx.data() + hq * hd;
      for (int i = lo; i <= pos; ++i) {                                               // src/kernels/mod.rs:494-506
        const float* vr = vat(l, kvh, i);
        for (int d = 0; d < hd; ++d) ch[d] += scores[i] * vr[d];
      }
    }
    matvec(L.wo.data(), ctx.data(), out.data(), H, nh * hd);                          // attention.rs:124-134
    for (int i = 0; i < H; ++i) h[i] += out[i];
    rmsnorm(h, L.n2.data(), c.eps, xn.data(), H);
    vector<float> g(I), u(I);
    matvec(L.wg.data(), xn.data(), g.data(), I, H);                                   // src/model/modules/mlp.rs:23-45
    matvec(L.wu.data(), xn.data(), u.data(), I, H);
    for (int i = 0; i < I; ++i) g[i] = silu(g[i]) * u[i];
    matvec(L.wd.data(), g.data(), out.data(), H, I);
    for (int i = 0; i < H; ++i) h[i] += out[i];
  }
  // src/model/mod.rs:430-447: embedding, layers, final norm, head.
  void forward(int token, int pos, float* logits) {
    vector<float> h(embed.begin() + (size_t)token * c.hidden, embed.begin() + (size_t)(token + 1) * c.hidden);
    for (int l = 0; l < c.layers; ++l) layer_forward(l, h.data(), pos);
    vector<float> xn(c.hidden);
    rmsnorm(h.data(), norm.data(), c.eps, xn.data(), c.hidden);
    matvec(head.data(), xn.data(), logits, c.vocab, c.hidden);
  }
  void make_inv_freq() {   // 1 / theta^(i / (hd/2)) (src/kernels/mod.rs:572-580)
    const int half = c.head_dim / 2;
    inv_freq.resize(half);
    for (int i = 0; i < half; ++i) inv_freq[i] = (float)(1.0 / pow((double)c.theta, (double)i / half));
  }
};

static Model load_model(const string& dir) {
  Model m;
  m.c = read_config(read_file(dir + "/config.json"));
  const Config& c = m.c;
  Weights w(dir + "/model.safetensors");
  const size_t H = c.hidden, Q = (size_t)c.heads * c.head_dim, KV = (size_t)c.kv_heads * c.head_dim, I = c.inter;
  m.embed = w.get("model.embed_tokens.weight", (size_t)c.vocab * H);   // names: src/model/mod.rs:360-414
  m.norm = w.get("model.norm.weight", H);
  m.head = w.get("lm_head.weight", (size_t)c.vocab * H);
  for (int l = 0; l < c.layers; ++l) {
    const string p = "model.layers." + std::to_string(l) + ".";
    Layer L;
    L.n1 = w.get(p + "input_layernorm.weight", H);
    L.n2 = w.get(p + "post_attention_layernorm.weight", H);
    L.wq = w.get(p + "self_attn.q_proj.weight", Q * H);
    L.wk = w.get(p + "self_attn.k_proj.weight", KV * H);
    L.wv = w.get(p + "self_attn.v_proj.weight", KV * H);
    L.wo = w.get(p + "self_attn.o_proj.weight", H * Q);
    L.wg = w.get(p + "mlp.gate_proj.weight", I * H);
    L.wu = w.get(p + "mlp.up_proj.weight", I * H);
    L.wd = w.get(p + "mlp.down_proj.weight", H * I);
    m.layers.push_back(std::move(L));
  }
  m.make_inv_freq();
  return m;
}

static double now() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
  if (argc == 5 && string(argv[1]) == "--time-layer") {
    Model m;
    m.c = read_config(read_file(argv[2]));
    const Config& c = m.c;
    const int context = atoi(argv[3]), repeats = atoi(argv[4]);
    const size_t H = c.hidden, Q = (size_t)c.heads * c.head_dim, KV = (size_t)c.kv_heads * c.head_dim, I = c.inter;
    uint32_t s = 12345;
    auto fill = [&](vector<float>& v, size_t n, float scale, float shift) {
      v.resize(n);
      for (size_t i = 0; i < n; ++i) { s = s * 1664525u + 1013904223u; v[i] = shift + scale * ((float)(s >> 8) / 8388608.0f - 1.0f); }
    };
    m.c.layers = 1;
    Layer L;
    fill(L.n1, H, 0.1f, 1.0f); fill(L.n2, H, 0.1f, 1.0f);
    fill(L.wq, Q * H, 0.03f, 0); fill(L.wk, KV * H, 0.03f, 0); fill(L.wv, KV * H, 0.03f, 0); fill(L.wo, H * Q, 0.03f, 0);
    fill(L.wg, I * H, 0.03f, 0); fill(L.wu, I * H, 0.03f, 0); fill(L.wd, H * I, 0.03f, 0);
    m.layers.push_back(std::move(L));
    fill(m.head, (size_t)c.vocab * H, 0.03f, 0);
    fill(m.norm, H, 0.1f, 1.0f);
    m.make_inv_freq();
    m.alloc_cache(context + repeats);
    fill(m.kc, m.kc.size(), 0.5f, 0); fill(m.vc, m.vc.size(), 0.5f, 0);
    vector<float> h, xn(H), logits(c.vocab);
    fill(h, H, 1.0f, 0);
    double t_layer = 1e30, t_head = 1e30;
    for (int r = 0; r < repeats; ++r) {
      vector<float> hh = h;
      double t0 = now();
      m.layer_forward(0, hh.data(), context + r);
      double t1 = now();
      rmsnorm(hh.data(), m.norm.data(), c.eps, xn.data(), (int)H);
      matvec(m.head.data(), xn.data(), logits.data(), c.vocab, (int)H);
      double t2 = now();
      if (t1 - t0 < t_layer) t_layer = t1 - t0;
      if (t2 - t1 < t_head) t_head = t2 - t1;
    }
    printf("{\"layer_s\": %.6f, \"head_s\": %.6f, \"context\": %d, \"checksum\": %.6g}\n", t_layer, t_head, context,
           (double)logits[0]);
    return 0;
  }
  if (argc != 4) die("usage: mistral_plain_onetoken <model_dir> <tokens.txt> <logits.f32>");
  Model m = load_model(argv[1]);
  vector<int> tokens;
  {
    std::ifstream f(argv[2]);
    int t;
    while (f >> t) tokens.push_back(t);
  }
  if (tokens.empty()) die("no tokens");
  m.alloc_cache((int)tokens.size());
  vector<float> logits((size_t)tokens.size() * m.c.vocab);
  for (size_t p = 0; p < tokens.size(); ++p) {
    if (tokens[p] < 0 || tokens[p] >= m.c.vocab) die("token id outside the vocabulary");
    m.forward(tokens[p], (int)p, logits.data() + p * m.c.vocab);
  }
  FILE* f = fopen(argv[3], "wb");
  if (!f) die(string("cannot write ") + argv[3]);
  fwrite(logits.data(), sizeof(float), logits.size(), f);
  fclose(f);
  return 0;
}
