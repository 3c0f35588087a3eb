// A second plain statement of the Llama / SmolLM2 decoder, in C++ and in the reference's own
// arithmetic: float32 values and sequential float32 sums with the float64 islands that
// martinsuchenak/scriptling-llm-lib has (each function cites file:line of the reference). The
// Python statement beside it (tests/plain_llama.py) computes everything in float64; this one shows
// that nothing in the tests hangs on that choice, and is written independently of it: whole
// sequences, no cache, one function per part. It shares no code with the library. The reference is
// Go and cannot be compiled where the tests run; nothing here was checked against its binary.
//
//   plain_llama MANIFEST WEIGHTS.f32 TOKENS.i32 OUT.f32
//
// MANIFEST (text): one "key value" line per configuration number (layers hidden heads kv_heads
// head_dim intermediate vocab rotary_dim eps theta interleaved tied window scaling_kind factor low
// high original), then one "tensor NAME OFFSET COUNT" line per tensor of WEIGHTS.f32 (float32,
// element offsets). TOKENS.i32: the sequence. OUT.f32: logits [S, vocab].
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

typedef std::vector<float> Vec;

struct Model {
  std::map<std::string, double> cfg;
  std::map<std::string, std::pair<size_t, size_t>> where;
  Vec data;
  const float* t(const std::string& name) const {
    auto it = where.find(name);
    if (it == where.end()) { fprintf(stderr, "no tensor %s\n", name.c_str()); exit(2); }
    return data.data() + it->second.first;
  }
  int i(const char* k) const { return (int)cfg.at(k); }
  double d(const char* k) const { return cfg.at(k); }
};

// rmsNormFlatF32, float32_ops.go:159-172: the sum of squares in float32, one after the other; the
// division, the eps and the square root in float64; y = (x * inv) * w in float32.
static void rms_norm(const float* x, const float* w, float* y, int rows, int d, double eps) {
  for (int r = 0; r < rows; r++) {
    float ss = 0.f;
    for (int j = 0; j < d; j++) ss += x[r * d + j] * x[r * d + j];
    float inv = (float)(1.0 / std::sqrt((double)ss / d + eps));
    for (int j = 0; j < d; j++) y[r * d + j] = (x[r * d + j] * inv) * w[j];
  }
}

// the dense product, float32_ops.go:462-482: y[r][j] = sum_l x[r][l] * W[j][l], float32, l ascending
static void linear(const float* x, const float* W, float* y, int rows, int in, int out) {
  for (int r = 0; r < rows; r++)
    for (int j = 0; j < out; j++) {
      float s = 0.f;
      for (int l = 0; l < in; l++) s += x[r * in + l] * W[(size_t)j * in + l];
      y[(size_t)r * out + j] = s;
    }
}

// the frequency table, model_f32.go:252-260: f_i = 1 / base^(2i / rotary_dim) in float64, kept as float32.
// The reference knows no rescaling; the llama3 and linear rules of the family's config.json rewrite the
// table (long wavelengths divided by the factor, short ones kept, the band between blended).
static std::vector<float> inv_freq(const Model& m) {
  int rot = m.i("rotary_dim");
  std::vector<float> f(rot / 2);
  const double pi = 3.14159265358979323846;
  for (int i = 0; i < rot / 2; i++) {
    double v = 1.0 / std::pow(m.d("theta"), 2.0 * i / rot);
    int kind = m.i("scaling_kind");                     // 0 none, 1 linear, 2 llama3
    if (kind == 1) v /= m.d("factor");
    if (kind == 2) {
      double wavelen = 2.0 * pi / v, orig = m.d("original");
      if (wavelen > orig / m.d("low")) v /= m.d("factor");
      else if (wavelen >= orig / m.d("high")) {
        double smooth = (orig / wavelen - m.d("low")) / (m.d("high") - m.d("low"));
        v = (1.0 - smooth) * v / m.d("factor") + smooth * v;
      }
    }
    f[i] = (float)v;
  }
  return f;
}

// applyRopeInPlaceF32, float32_ops.go:174-188: the angle f_i * position in float32, its cosine and
// sine in float64 cast to float32, the rotation in float32; dims past the rotary width untouched.
// Adjacent pairs as in the reference, or pairs (i, i + width/2) as checkpoints of the family have them.
static void rope(float* x, int S, int heads, int hd, const std::vector<float>& f, bool interleaved) {
  int half = (int)f.size();
  for (int p = 0; p < S; p++)
    for (int h = 0; h < heads; h++) {
      float* v = x + ((size_t)p * heads + h) * hd;
      for (int i = 0; i < half; i++) {
        float theta = f[i] * (float)p;
        float c = (float)std::cos((double)theta), s = (float)std::sin((double)theta);
        int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
        float a = v[i0], b = v[i1];
        v[i0] = a * c - b * s;
        v[i1] = a * s + b * c;
      }
    }
}

// fusedAttentionHeadF32, float32_ops.go:190-235, with the grouping of :252-260 (query head h reads
// key/value head h / (H / G)): score = dot * (1/sqrt(hd)) after the dot product, keys after the query
// masked (and, with a window, keys `window` or more behind it), max-subtracted softmax whose
// exponential is taken in float64 on the float32 difference, out = sum (e * (1/Z)) * v in float32.
static void attention(const float* q, const float* k, const float* v, float* out, int S, int H, int G, int hd, int window) {
  float scale = (float)(1.0 / std::sqrt((double)hd));
  std::vector<float> sc(S), e(S);
  for (int h = 0; h < H; h++) {
    int g = h / (H / G);
    for (int qi = 0; qi < S; qi++) {
      int lo = window > 0 ? std::max(0, qi - window + 1) : 0;
      float mx = -INFINITY;
      for (int kj = lo; kj <= qi; kj++) {
        float dot = 0.f;
        for (int dd = 0; dd < hd; dd++) dot += q[((size_t)qi * H + h) * hd + dd] * k[((size_t)kj * G + g) * hd + dd];
        sc[kj] = dot * scale;
        mx = std::max(mx, sc[kj]);
      }
      float Z = 0.f;
      for (int kj = lo; kj <= qi; kj++) { e[kj] = (float)std::exp((double)(sc[kj] - mx)); Z += e[kj]; }
      float invZ = 1.0f / Z;
      for (int dd = 0; dd < hd; dd++) {
        float o = 0.f;
        for (int kj = lo; kj <= qi; kj++) o += (e[kj] * invZ) * v[((size_t)kj * G + g) * hd + dd];
        out[((size_t)qi * H + h) * hd + dd] = o;
      }
    }
  }
}

int main(int argc, char** argv) {
  if (argc != 5) { fprintf(stderr, "usage: plain_llama MANIFEST WEIGHTS.f32 TOKENS.i32 OUT.f32\n"); return 1; }
  Model m;
  std::ifstream mf(argv[1]);
  std::string line;
  while (std::getline(mf, line)) {
    std::istringstream ls(line);
    std::string key;
    ls >> key;
    if (key == "tensor") { std::string name; size_t off, n; ls >> name >> off >> n; m.where[name] = {off, n}; }
    else if (!key.empty()) { double v; ls >> v; m.cfg[key] = v; }
  }
  { std::ifstream wf(argv[2], std::ios::binary | std::ios::ate); size_t bytes = wf.tellg(); wf.seekg(0);
    m.data.resize(bytes / 4); wf.read((char*)m.data.data(), bytes); }
  std::vector<int> ids;
  { std::ifstream tf(argv[3], std::ios::binary | std::ios::ate); size_t bytes = tf.tellg(); tf.seekg(0);
    ids.resize(bytes / 4); tf.read((char*)ids.data(), bytes); }
  const int S = (int)ids.size(), L = m.i("layers"), d = m.i("hidden"), H = m.i("heads"), G = m.i("kv_heads"), hd = m.i("head_dim"),
            F = m.i("intermediate"), V = m.i("vocab"), window = m.i("window");
  const double eps = m.d("eps");
  const bool interleaved = m.i("interleaved") != 0;
  std::vector<float> f = inv_freq(m);

  Vec x((size_t)S * d), n((size_t)S * d), q((size_t)S * H * hd), k((size_t)S * G * hd), v((size_t)S * G * hd), a((size_t)S * H * hd),
      o((size_t)S * d), gate((size_t)S * F), up((size_t)S * F), hmid((size_t)S * F), down((size_t)S * d);
  const float* E = m.t("model.embed_tokens.weight");
  for (int p = 0; p < S; p++)                                  // model_f32.go:363-369: a copy, no scaling
    for (int j = 0; j < d; j++) x[(size_t)p * d + j] = E[(size_t)ids[p] * d + j];
  for (int l = 0; l < L; l++) {                                // model_f32.go:382-500
    std::string p = "model.layers." + std::to_string(l) + ".";
    rms_norm(x.data(), m.t(p + "input_layernorm.weight"), n.data(), S, d, eps);
    linear(n.data(), m.t(p + "self_attn.q_proj.weight"), q.data(), S, d, H * hd);
    linear(n.data(), m.t(p + "self_attn.k_proj.weight"), k.data(), S, d, G * hd);
    linear(n.data(), m.t(p + "self_attn.v_proj.weight"), v.data(), S, d, G * hd);
    rope(q.data(), S, H, hd, f, interleaved);
    rope(k.data(), S, G, hd, f, interleaved);
    attention(q.data(), k.data(), v.data(), a.data(), S, H, G, hd, window);
    linear(a.data(), m.t(p + "self_attn.o_proj.weight"), o.data(), S, H * hd, d);
    for (size_t i = 0; i < x.size(); i++) x[i] += o[i];        // model_f32.go:472-474
    rms_norm(x.data(), m.t(p + "post_attention_layernorm.weight"), n.data(), S, d, eps);
    linear(n.data(), m.t(p + "mlp.gate_proj.weight"), gate.data(), S, d, F);
    linear(n.data(), m.t(p + "mlp.up_proj.weight"), up.data(), S, d, F);
    for (size_t i = 0; i < hmid.size(); i++) {                 // model_f32.go:484-490: the sigmoid in float64, g * s * u left to right
      float sg = (float)(1.0 / (1.0 + std::exp(-(double)gate[i])));
      hmid[i] = gate[i] * sg * up[i];
    }
    linear(hmid.data(), m.t(p + "mlp.down_proj.weight"), down.data(), S, F, d);
    for (size_t i = 0; i < x.size(); i++) x[i] += down[i];     // model_f32.go:495-497
  }
  rms_norm(x.data(), m.t("model.norm.weight"), n.data(), S, d, eps);          // model_f32.go:502-517 (there: the last row only)
  const float* head = m.i("tied") ? E : m.t("lm_head.weight");                 // model_f32.go:147-162, :519-524
  Vec logits((size_t)S * V);
  linear(n.data(), head, logits.data(), S, d, V);
  std::ofstream of(argv[4], std::ios::binary);
  of.write((const char*)logits.data(), logits.size() * 4);
  return 0;
}
