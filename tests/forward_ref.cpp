// forward_ref: a second plain implementation of LFM2, in C++ and 32-bit floats, for the tests.
//
// It follows the shape of pylypenko99/zinfer's own engine rather than that of the NumPy oracle
// beside it (tests/plain_lfm2.py, which evaluates whole sequences without any cache): one
// sequence with a position counter, a key/value cache per attention layer, a convolution state
// per conv layer, and a `forward(tokens)` that runs the given tokens from that state and moves
// the position on (State.forwardBatch, src/model.zig:2347-2516).  The two share nothing: this
// file has its own safetensors reader, takes every size from the tensors' shapes the way zinfer
// takes them from its file (src/model.zig:408-508), and is written from the cited lines.
// Neither rests on a run of zinfer (no Zig compiler is at hand); the tests check that they agree.
//
// Differences from zinfer's arithmetic, on purpose: `expf` from the C library instead of the
// degree-6 polynomial (src/ffn.zig:12-28), no skipped softmax tiles (src/attention.zig:493), and
// keys and values kept in float32 instead of float16 (src/model.zig:1915-1922).
//
// C interface (loaded with ctypes):
//   ref_open(path to model.safetensors, eps, rope theta, window per layer [n_layers] or null, max positions)
//   ref_forward(state, tokens, n, logits out [n, vocab])   runs n more tokens, logits of all of them
//   ref_reset(state)   back to position 0 with empty caches;  ref_close(state)
//   ref_vocab / ref_layers / ref_error
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace {

std::string g_error;

struct Tensor {
  std::vector<int64_t> shape;
  std::vector<float> data;
  int64_t rows() const { return shape.empty() ? 0 : shape[0]; }
  int64_t cols() const {
    int64_t n = 1;
    for (size_t i = 1; i < shape.size(); ++i) n *= shape[i];
    return n;
  }
};

// ------------------------------------------------------------------ the container
// 8 bytes little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, raw data.

struct Cursor {
  const char* p;
  const char* end;
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < end && *p == c) {
      ++p;
      return true;
    }
    return false;
  }
  bool str(std::string* out) {
    ws();
    if (p >= end || *p != '"') return false;
    ++p;
    out->clear();
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) ++p;
      out->push_back(*p++);
    }
    if (p >= end) return false;
    ++p;
    return true;
  }
  bool integer(int64_t* out) {
    ws();
    const char* s = p;
    int64_t v = 0;
    while (p < end && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
    *out = v;
    return p > s;
  }
  bool int_list(std::vector<int64_t>* out) {
    out->clear();
    if (!eat('[')) return false;
    if (eat(']')) return true;
    do {
      int64_t v;
      if (!integer(&v)) return false;
      out->push_back(v);
    } while (eat(','));
    return eat(']');
  }
  bool skip_value() {  // strings, numbers, objects, lists, literals
    ws();
    if (p >= end) return false;
    if (*p == '"') {
      std::string s;
      return str(&s);
    }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (eat(close)) return true;
      do {
        if (open == '{') {
          std::string k;
          if (!str(&k) || !eat(':')) return false;
        }
        if (!skip_value()) return false;
      } while (eat(','));
      return eat(close);
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;
    return true;
  }
};

float bf16_to_float(uint16_t h) {
  const uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

float f16_to_float(uint16_t h) {
  const int sign = h >> 15, e = (h >> 10) & 31, m = h & 1023;
  float v;
  if (e == 0) v = std::ldexp((float)m, -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = std::ldexp((float)(m | 1024), e - 25);
  return sign ? -v : v;
}

bool read_file(const char* path, std::map<std::string, Tensor>* out) {
  FILE* f = fopen(path, "rb");
  if (!f) return g_error = std::string("cannot open ") + path, false;
  std::vector<char> raw;
  fseek(f, 0, SEEK_END);
  const long size = ftell(f);
  fseek(f, 0, SEEK_SET);
  raw.resize((size_t)size);
  const size_t got = fread(raw.data(), 1, raw.size(), f);
  fclose(f);
  if (got != raw.size() || raw.size() < 8) return g_error = "short file", false;
  uint64_t hlen = 0;
  memcpy(&hlen, raw.data(), 8);
  if (8 + hlen > raw.size()) return g_error = "header longer than the file", false;
  const char* base = raw.data() + 8 + hlen;
  const size_t data_size = raw.size() - 8 - (size_t)hlen;
  Cursor c{raw.data() + 8, raw.data() + 8 + hlen};
  if (!c.eat('{')) return g_error = "header is no object", false;
  if (c.eat('}')) return true;
  do {
    std::string name;
    if (!c.str(&name) || !c.eat(':')) return g_error = "bad header", false;
    if (name == "__metadata__") {
      if (!c.skip_value()) return g_error = "bad metadata", false;
      continue;
    }
    if (!c.eat('{')) return g_error = "bad tensor entry", false;
    std::string dtype;
    std::vector<int64_t> shape, offs;
    do {
      std::string key;
      if (!c.str(&key) || !c.eat(':')) return g_error = "bad tensor entry", false;
      bool ok = key == "dtype" ? c.str(&dtype) : key == "shape" ? c.int_list(&shape)
                : key == "data_offsets" ? c.int_list(&offs) : c.skip_value();
      if (!ok) return g_error = "bad tensor entry " + name, false;
    } while (c.eat(','));
    if (!c.eat('}') || offs.size() != 2) return g_error = "bad tensor entry " + name, false;
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    const int width = dtype == "F32" ? 4 : (dtype == "BF16" || dtype == "F16") ? 2 : 0;
    if (!width) return g_error = "dtype " + dtype + " of " + name, false;
    if (offs[1] - offs[0] != n * width || (size_t)offs[1] > data_size) return g_error = "bad offsets of " + name, false;
    Tensor t;
    t.shape = shape;
    t.data.resize((size_t)n);
    const char* src = base + offs[0];
    for (int64_t i = 0; i < n; ++i) {
      if (width == 4) memcpy(&t.data[i], src + 4 * i, 4);
      else {
        uint16_t h;
        memcpy(&h, src + 2 * i, 2);
        t.data[i] = dtype == "BF16" ? bf16_to_float(h) : f16_to_float(h);
      }
    }
    (*out)[name] = std::move(t);
  } while (c.eat(','));
  return true;
}

// ------------------------------------------------------------------ the model

struct Layer {
  bool conv = false;
  const Tensor *mix_norm = nullptr, *ffn_norm = nullptr;
  // short convolution (src/model.zig:729-734)
  const Tensor *in_proj = nullptr, *taps = nullptr, *out_proj = nullptr, *conv_bias = nullptr, *in_bias = nullptr, *out_bias = nullptr;
  int n_taps = 0;
  // attention (src/model.zig:756-776)
  const Tensor *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  int n_heads = 0, n_kv = 0, hd = 0, window = 0;
  // feed-forward (src/model.zig:712-717)
  const Tensor *w_gate = nullptr, *w_up = nullptr, *w_down = nullptr;
  // state of the one sequence
  std::vector<float> k_cache, v_cache;   // [position][kv head][hd]
  std::vector<float> conv_state;         // [taps - 1][dim], the last conv inputs (src/model.zig:1502)
};

struct State {
  std::map<std::string, Tensor> w;
  std::vector<Layer> layers;
  const Tensor *embd = nullptr, *out_norm = nullptr, *output = nullptr;
  int dim = 0, vocab = 0, max_pos = 0;
  float eps = 1e-5f, theta = 10000.f;
  int pos = 0;
  std::vector<float> freqs;   // [hd / 2]
};

const Tensor* find(State* s, const std::string& name) {
  auto it = s->w.find(name);
  return it == s->w.end() ? nullptr : &it->second;
}

// y = x * 1/sqrt(mean(x^2) + eps) * w: scale first, weight second (src/model.zig:1166-1181)
void rmsnorm(float* out, const float* x, const float* w, int n, float eps) {
  float ss = 0.f;
  for (int i = 0; i < n; ++i) ss += x[i] * x[i];
  const float scale = 1.0f / std::sqrt(ss / (float)n + eps);
  for (int i = 0; i < n; ++i) out[i] = x[i] * scale * w[i];
}

// out[r] (+)= sum_c W[r][c] * x[c] (+ bias[r])   (the matmul driver, src/model.zig:903-1026; accumulate: 918-920)
void matvec(float* out, const Tensor* W, const float* x, bool accumulate, const Tensor* bias = nullptr) {
  const int64_t R = W->rows(), C = W->cols();
  for (int64_t r = 0; r < R; ++r) {
    const float* row = &W->data[(size_t)(r * C)];
    float acc = 0.f;
    for (int64_t c = 0; c < C; ++c) acc += row[c] * x[c];
    if (bias) acc += bias->data[(size_t)r];
    out[r] = accumulate ? out[r] + acc : acc;
  }
}

// f_i = theta^(-2i / n_rot), in double, cast to float (src/rope.zig:8-16)
void rope_freqs(State* s, int hd) {
  s->freqs.resize((size_t)hd / 2);
  for (int i = 0; i < hd / 2; ++i) {
    const double e = -2.0 * (double)i / (double)hd;
    s->freqs[(size_t)i] = (float)std::pow((double)s->theta, e);
  }
}

// NeoX pairing (i, i + half); angle = float(pos) * f_i as a float product (src/rope.zig:34-45, 50-64;
// NeoX for every architecture but llama, src/model.zig:449)
void rope(float* v, int n_heads, int hd, int pos, const std::vector<float>& freqs) {
  const int half = hd / 2;
  for (int h = 0; h < n_heads; ++h) {
    float* x = v + (size_t)h * hd;
    for (int i = 0; i < half; ++i) {
      const float a = (float)pos * freqs[(size_t)i];
      const float cs = std::cos(a), sn = std::sin(a);
      const float p = x[i], q = x[i + half];
      x[i] = p * cs - q * sn;
      x[i + half] = p * sn + q * cs;
    }
  }
}

// [B, C, X] = W_in xn; u = B * X; y = C * sum_k w[k] * hist[t + k] with the state in front of the new
// rows; the state becomes the last taps - 1 rows; x += W_out y (src/model.zig:1994-2028)
void short_conv(State* s, Layer& L, const std::vector<float>& xn, int nt, std::vector<float>& x) {
  const int d = s->dim, taps = L.n_taps, hist = taps - 1;
  std::vector<float> bcx((size_t)3 * d), rows((size_t)(hist + nt) * d), y((size_t)d);
  memcpy(rows.data(), L.conv_state.data(), sizeof(float) * (size_t)hist * d);
  std::vector<float> cgate((size_t)nt * d);
  for (int t = 0; t < nt; ++t) {
    matvec(bcx.data(), L.in_proj, &xn[(size_t)t * d], false, L.in_bias);
    for (int ch = 0; ch < d; ++ch) {
      rows[(size_t)(hist + t) * d + ch] = bcx[(size_t)ch] * bcx[(size_t)2 * d + ch];
      cgate[(size_t)t * d + ch] = bcx[(size_t)d + ch];
    }
  }
  for (int t = 0; t < nt; ++t) {
    for (int ch = 0; ch < d; ++ch) {
      float acc = 0.f;
      // the file holds taps as [channel][1][tap]; zinfer turns them to [tap][channel] (src/model.zig:788-802)
      for (int k = 0; k < taps; ++k) acc = std::fma(L.taps->data[(size_t)ch * taps + k], rows[(size_t)(t + k) * d + ch], acc);
      if (L.conv_bias) acc += L.conv_bias->data[(size_t)ch];   // this build's extension; zinfer has no conv bias
      y[(size_t)ch] = acc * cgate[(size_t)t * d + ch];
    }
    matvec(&x[(size_t)t * d], L.out_proj, y.data(), true, L.out_bias);
  }
  memcpy(L.conv_state.data(), &rows[(size_t)nt * d], sizeof(float) * (size_t)hist * d);
}

// q, k, v; per-head RMSNorm of q and k before the rotation (src/model.zig:1741-1744, 1760-1763); keys and
// values stored at their absolute positions; every query sees keys [lo, pos] with lo = pos + 1 - window
// when a window is set (src/model.zig:1360-1363); query head h reads KV head h / (H / Hkv)
// (src/model.zig:1330, 1352-1366); scores scaled by 1/sqrt(hd) (src/model.zig:465); x += W_o att
void attention(State* s, Layer& L, const std::vector<float>& xn, int nt, std::vector<float>& x) {
  const int d = s->dim, H = L.n_heads, Hkv = L.n_kv, hd = L.hd, g = H / Hkv;
  const int q_dim = H * hd, kv_dim = Hkv * hd;
  const float scale = 1.0f / std::sqrt((float)hd);
  std::vector<float> q((size_t)q_dim), k((size_t)kv_dim), v((size_t)kv_dim), att((size_t)q_dim), sc;
  for (int t = 0; t < nt; ++t) {
    const int p = s->pos + t;
    matvec(q.data(), L.wq, &xn[(size_t)t * d], false);
    matvec(k.data(), L.wk, &xn[(size_t)t * d], false);
    matvec(v.data(), L.wv, &xn[(size_t)t * d], false);
    for (int h = 0; h < H; ++h) rmsnorm(&q[(size_t)h * hd], &q[(size_t)h * hd], L.q_norm->data.data(), hd, s->eps);
    for (int h = 0; h < Hkv; ++h) rmsnorm(&k[(size_t)h * hd], &k[(size_t)h * hd], L.k_norm->data.data(), hd, s->eps);
    rope(q.data(), H, hd, p, s->freqs);
    rope(k.data(), Hkv, hd, p, s->freqs);
    memcpy(&L.k_cache[(size_t)p * kv_dim], k.data(), sizeof(float) * (size_t)kv_dim);
    memcpy(&L.v_cache[(size_t)p * kv_dim], v.data(), sizeof(float) * (size_t)kv_dim);
    const int np = p + 1;
    const int lo = (L.window > 0 && np > L.window) ? np - L.window : 0;
    sc.resize((size_t)(np - lo));
    for (int h = 0; h < H; ++h) {
      const int kh = h / g;
      float m = -INFINITY;
      for (int j = lo; j < np; ++j) {
        const float* kj = &L.k_cache[(size_t)j * kv_dim + (size_t)kh * hd];
        float dot = 0.f;
        for (int i = 0; i < hd; ++i) dot += q[(size_t)h * hd + i] * kj[i];
        sc[(size_t)(j - lo)] = dot * scale;
        m = std::fmax(m, dot * scale);
      }
      float l = 0.f;
      for (int j = lo; j < np; ++j) {
        sc[(size_t)(j - lo)] = std::exp(sc[(size_t)(j - lo)] - m);
        l += sc[(size_t)(j - lo)];
      }
      for (int i = 0; i < hd; ++i) {
        float o = 0.f;
        for (int j = lo; j < np; ++j) o += sc[(size_t)(j - lo)] * L.v_cache[(size_t)j * kv_dim + (size_t)kh * hd + i];
        att[(size_t)h * hd + i] = l > 0.f ? o / l : 0.f;
      }
    }
    matvec(&x[(size_t)t * d], L.wo, att.data(), true);
  }
}

// h = silu(W_gate xn) * (W_up xn), silu(g) = g / (1 + exp(-g)) (src/ffn.zig:31-33, 49-57); x += W_down h
void feed_forward(State* s, Layer& L, const std::vector<float>& xn, int nt, std::vector<float>& x) {
  const int d = s->dim, F = (int)L.w_gate->rows();
  std::vector<float> gt((size_t)F), up((size_t)F);
  for (int t = 0; t < nt; ++t) {
    matvec(gt.data(), L.w_gate, &xn[(size_t)t * d], false);
    matvec(up.data(), L.w_up, &xn[(size_t)t * d], false);
    for (int i = 0; i < F; ++i) gt[(size_t)i] = gt[(size_t)i] / (1.0f + std::exp(-gt[(size_t)i])) * up[(size_t)i];
    matvec(&x[(size_t)t * d], L.w_down, gt.data(), true);
  }
}

bool bind(State* s, const int* windows) {
  s->embd = find(s, "model.embed_tokens.weight");
  s->out_norm = find(s, "model.embedding_norm.weight");   // LFM2's final norm is the embedding norm (src/model.zig:599-600)
  if (!s->embd || !s->out_norm) return g_error = "no embedding or final norm", false;
  s->output = find(s, "lm_head.weight");
  if (!s->output) s->output = s->embd;                    // tied when the tensor is absent (src/model.zig:595-598)
  s->vocab = (int)s->embd->rows();
  s->dim = (int)s->embd->cols();
  for (int i = 0;; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    Layer L;
    L.mix_norm = find(s, p + "operator_norm.weight");
    if (!L.mix_norm) break;
    L.ffn_norm = find(s, p + "ffn_norm.weight");
    L.w_gate = find(s, p + "feed_forward.w1.weight");
    L.w_up = find(s, p + "feed_forward.w3.weight");
    L.w_down = find(s, p + "feed_forward.w2.weight");
    if (!L.ffn_norm || !L.w_gate || !L.w_up || !L.w_down) return g_error = "layer without a feed-forward", false;
    L.in_proj = find(s, p + "conv.in_proj.weight");
    if (L.in_proj) {
      L.conv = true;
      L.taps = find(s, p + "conv.conv.weight");
      L.out_proj = find(s, p + "conv.out_proj.weight");
      if (!L.taps || !L.out_proj) return g_error = "conv layer without taps or out_proj", false;
      L.conv_bias = find(s, p + "conv.conv.bias");
      L.in_bias = find(s, p + "conv.in_proj.bias");
      L.out_bias = find(s, p + "conv.out_proj.bias");
      L.n_taps = (int)(L.taps->cols());
      if (L.n_taps < 2) return g_error = "a conv layer needs at least 2 taps", false;   // src/model.zig:486
      L.conv_state.assign((size_t)(L.n_taps - 1) * s->dim, 0.f);
    } else {
      const std::string a = p + "self_attn.";
      L.wq = find(s, a + "q_proj.weight");
      L.wk = find(s, a + "k_proj.weight");
      L.wv = find(s, a + "v_proj.weight");
      L.wo = find(s, a + "out_proj.weight");
      L.q_norm = find(s, a + "q_layernorm.weight");
      L.k_norm = find(s, a + "k_layernorm.weight");
      if (!L.wq || !L.wk || !L.wv || !L.wo || !L.q_norm || !L.k_norm) return g_error = "layer " + std::to_string(i) + " has no mixer", false;
      L.hd = (int)L.q_norm->rows();
      L.n_heads = (int)L.wq->rows() / L.hd;
      L.n_kv = (int)L.wk->rows() / L.hd;
      if (L.n_heads % L.n_kv) return g_error = "heads are no multiple of KV heads", false;   // src/model.zig:487
      L.window = windows ? windows[i] : 0;
      L.k_cache.assign((size_t)s->max_pos * L.n_kv * L.hd, 0.f);
      L.v_cache.assign((size_t)s->max_pos * L.n_kv * L.hd, 0.f);
      if (s->freqs.empty()) rope_freqs(s, L.hd);
    }
    s->layers.push_back(std::move(L));
  }
  return !s->layers.empty() || (g_error = "no layers", false);
}

}  // namespace

extern "C" {

const char* ref_error() { return g_error.c_str(); }

void* ref_open(const char* path, float eps, float theta, const int* windows, int max_positions) {
  State* s = new State;
  s->eps = eps;
  s->theta = theta;
  s->max_pos = max_positions;
  if (!read_file(path, &s->w) || !bind(s, windows)) {
    delete s;
    return nullptr;
  }
  return s;
}

void ref_close(void* st) { delete static_cast<State*>(st); }
int ref_vocab(void* st) { return static_cast<State*>(st)->vocab; }
int ref_layers(void* st) { return (int)static_cast<State*>(st)->layers.size(); }

void ref_reset(void* st) {
  State* s = static_cast<State*>(st);
  s->pos = 0;
  for (Layer& L : s->layers) std::fill(L.conv_state.begin(), L.conv_state.end(), 0.f);   // src/model.zig:1617-1621
}

// Runs `n` more tokens of the sequence; logits [n, vocab] of all of them.  Returns 0, or -1 when the
// context is full (src/model.zig:2520) or a token lies outside the vocabulary.
int ref_forward(void* st, const int* tokens, int n, float* logits) {
  State* s = static_cast<State*>(st);
  const int d = s->dim;
  if (s->pos + n > s->max_pos) return g_error = "context full", -1;
  std::vector<float> x((size_t)n * d), xn((size_t)n * d);
  for (int t = 0; t < n; ++t) {
    if (tokens[t] < 0 || tokens[t] >= s->vocab) return g_error = "token outside the vocabulary", -1;
    memcpy(&x[(size_t)t * d], &s->embd->data[(size_t)tokens[t] * d], sizeof(float) * (size_t)d);   // src/model.zig:2352-2358
  }
  for (Layer& L : s->layers) {   // x += Mixer(norm(x)); x += FFN(norm(x))   (src/model.zig:2395-2422)
    for (int t = 0; t < n; ++t) rmsnorm(&xn[(size_t)t * d], &x[(size_t)t * d], L.mix_norm->data.data(), d, s->eps);
    if (L.conv) short_conv(s, L, xn, n, x);
    else attention(s, L, xn, n, x);
    for (int t = 0; t < n; ++t) rmsnorm(&xn[(size_t)t * d], &x[(size_t)t * d], L.ffn_norm->data.data(), d, s->eps);
    feed_forward(s, L, xn, n, x);
  }
  s->pos += n;   // src/model.zig:2480
  for (int t = 0; t < n; ++t) {   // src/model.zig:2482-2490
    rmsnorm(&xn[(size_t)t * d], &x[(size_t)t * d], s->out_norm->data.data(), d, s->eps);
    matvec(logits + (size_t)t * s->vocab, s->output, &xn[(size_t)t * d], false);
  }
  return 0;
}

}  // extern "C"
