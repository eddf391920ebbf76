// CPU oracle for the Llama-3 forward path of NFAI -- TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the CPU, the arithmetic that the reference performs in its nine GLSL compute
// shaders and in the host code between them. It is the checker for the CUDA library; it is never part of
// the product path. Only the tests, the smoke check and the CPU-baseline / reference legs of the benchmark
// may load it.
//
// PARITY UNPINNED: the reference ships no tests, golden vectors or fixtures for this path, and it cannot be
// run where this oracle is built (C#/.NET + Vulkan + glslangValidator). The GLSL built-ins exp/sin/cos/sqrt
// have driver-defined precision, so the values below (libm, float32) define the target.
//
// Each function cites the reference lines it follows (paths relative to the reference project root).
// Arithmetic is float32 with the loops in the shaders' index order; build with -ffp-contract=off so that
// a*b+c is two roundings (the defined mode). Mode 1 accumulates every reduction in double and rounds once;
// it is used to tell an ordering difference from a bug when two logits are nearly tied.
//
// Documented divergences from the literal reference (the oracle implements the intended math):
//  * RoPE is applied to every pair m < ropeDim/2 of every head, with the full frequency table
//    (the reference uploads a table of hard-coded length 32: NFAI.Vulkan.Shaders/TransformerBlock.cs:66).
//  * Scores are computed race-free for t <= p only (the reference also writes -1e9 fills that alias other
//    heads' rows: NFAI.Vulkan.Shaders/AttentionScoreCalculationShader.cs:180-184).
//  * An untied LM head (output.weight) is used when present; the reference always ties
//    (NFAI.Models.Llama3/LlamaModel.cs:64-67).
//  * A position >= ctx is an error instead of an out-of-bounds write.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__F16C__)
#include <immintrin.h>
#endif

extern "C" {

typedef struct {
  uint32_t H, L, qH, kvH, d, ropeDim, F, V, ctx;
  float eps;
  float rope_theta;
  int32_t mode;  // 0 = float32 sequential (defined mode), 1 = double accumulation
} orc_hparams;

}  // extern "C"

namespace {

// Exact binary16 -> binary32 widening; same value as C#'s (float)Half used at
// NFAI.Core/AbstractComputeCollection.cs:62-77 (and the bit-level helper at :81-131).
inline float half_to_float(uint16_t h) {
#if defined(__F16C__)
  return _cvtsh_ss(h);
#else
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int shift = 0;
      while ((man & 0x400) == 0) { man <<= 1; ++shift; }
      man &= 0x3FF;
      bits = sign | (uint32_t)(1 - shift + 127 - 15) << 23 | man << 13;
    }
  } else if (exp == 0x1F) {
    bits = sign | 0xFFu << 23 | man << 13;
  } else {
    bits = sign | (exp + 127 - 15) << 23 | man << 13;
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
#endif
}

struct Tensor {
  int dtype = -1;  // 0 f32, 1 f16
  uint64_t count = 0;
  std::vector<float> f32;
  std::vector<uint16_t> f16;
  bool present() const { return dtype >= 0; }
  inline float at(uint64_t i) const { return dtype == 0 ? f32[i] : half_to_float(f16[i]); }
};

struct Layer {
  Tensor attn_norm, wq, wk, wv, wo, ffn_norm, wgate, wup, wdown;
};

struct Model {
  orc_hparams hp;
  Tensor embd, out_norm, out_head;
  std::vector<Layer> layers;
  std::vector<float> kc, vc;        // [L][ctx][kvDim]
  std::vector<float> rope_f;        // [ropeDim/2]
  std::vector<float> hidden_taps;   // [L][H] block outputs of the last step
  std::vector<float> last_q;        // [L][qDim] rotated queries of the last step
  std::vector<float> last_attn;     // [L][qDim] attention outputs of the last step
  uint32_t pos = 0;
  std::string err;
};

// y[j] = sum_k x[k] * W[j*K + k], k ascending, float32 (NFAI.Vulkan.Shaders/MatrixMultiplyShader.cs:266-288,
// "transpose" index form j*inputCols+k at :260). Rows are independent, so they run in parallel; eight rows
// are interleaved per thread only to hide the add latency -- each row's own order is untouched.
template <typename LoadW>
void matvec_rows(const float* x, LoadW w, uint64_t K, uint64_t N, float* y, int mode) {
  const int64_t nblk = (int64_t)((N + 7) / 8);
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nblk; ++b) {
    uint64_t j0 = (uint64_t)b * 8;
    int nr = (int)((N - j0) < 8 ? (N - j0) : 8);
    if (mode == 0) {
      float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (nr == 8) {
        for (uint64_t k = 0; k < K; ++k) {
          float xv = x[k];
          for (int r = 0; r < 8; ++r) s[r] += xv * w((j0 + r) * K + k);
        }
      } else {
        for (uint64_t k = 0; k < K; ++k) {
          float xv = x[k];
          for (int r = 0; r < nr; ++r) s[r] += xv * w((j0 + r) * K + k);
        }
      }
      for (int r = 0; r < nr; ++r) y[j0 + r] = s[r];
    } else {
      double s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (uint64_t k = 0; k < K; ++k) {
        double xv = x[k];
        for (int r = 0; r < nr; ++r) s[r] += xv * (double)w((j0 + r) * K + k);
      }
      for (int r = 0; r < nr; ++r) y[j0 + r] = (float)s[r];
    }
  }
}

void matvec(const float* x, const Tensor& W, uint64_t K, uint64_t N, float* y, int mode) {
  if (W.dtype == 0) {
    const float* p = W.f32.data();
    matvec_rows(x, [p](uint64_t i) { return p[i]; }, K, N, y, mode);
  } else {
    const uint16_t* p = W.f16.data();
    matvec_rows(x, [p](uint64_t i) { return half_to_float(p[i]); }, K, N, y, mode);
  }
}

// NFAI.Vulkan.Shaders/RMSNormShader.cs:129-150: sumSq sequential, meanSq = sumSq/float(H),
// rms = sqrt(meanSq + eps), out = (x / rms) * gamma.
void rmsnorm(const float* x, const Tensor& g, uint32_t H, float eps, float* y, int mode) {
  float meanSq;
  if (mode == 0) {
    float ss = 0.0f;
    for (uint32_t i = 0; i < H; ++i) ss += x[i] * x[i];
    meanSq = ss / (float)H;
  } else {
    double ss = 0.0;
    for (uint32_t i = 0; i < H; ++i) ss += (double)x[i] * (double)x[i];
    meanSq = (float)(ss / (double)H);
  }
  float rms = sqrtf(meanSq + eps);
  for (uint32_t i = 0; i < H; ++i) y[i] = (x[i] / rms) * g.at(i);
}

// Frequency table: NFAI.Vulkan.Shaders/TransformerBlock.cs:33-38, float32 powf and division.
void rope_table(uint32_t ropeDim, float theta_base, std::vector<float>& f) {
  f.resize(ropeDim / 2);
  for (uint32_t i = 0; i < ropeDim / 2; ++i)
    f[i] = 1.0f / powf(theta_base, (float)i / ((float)ropeDim / 2));
}

// NFAI.Vulkan.Shaders/RoPEShader.cs:238-271: adjacent pairs (2m, 2m+1), theta = f[m]*float(pos),
// v1 = c*a - s*b, v2 = s*a + c*b; elements beyond ropeDim are copied unchanged. In place.
void rope(float* v, uint32_t heads, uint32_t d, uint32_t ropeDim, const float* f, uint32_t pos) {
  for (uint32_t h = 0; h < heads; ++h)
    for (uint32_t m = 0; 2 * m + 1 < d && 2 * m < ropeDim; ++m) {
      float theta = f[m] * (float)pos;
      float c = cosf(theta), s = sinf(theta);
      float a = v[h * d + 2 * m], b = v[h * d + 2 * m + 1];
      v[h * d + 2 * m] = c * a - s * b;
      v[h * d + 2 * m + 1] = s * a + c * b;
    }
}

// Scores, clamped softmax and weighted value sum for one new token over positions 0..seq-1:
// NFAI.Vulkan.Shaders/AttentionScoreCalculationShader.cs:170-205 (dot over i ascending, times 1/sqrt(d),
// kvHead = qHead / (qH/kvH)), AttentionSoftmaxShader.cs:145-177 (max from -1e38, exp(clamp(s-max,-80,80)),
// inv = sum > eps ? 1/sum : 0) and AttentionWeightedValueSumShader.cs:181-215 (t ascending).
void attention(const float* q, const float* kc, const float* vc, uint32_t seq, uint32_t qH, uint32_t kvH,
               uint32_t d, float eps, float* out, int mode) {
  const uint32_t kvDim = kvH * d;
  const float scale = 1.0f / sqrtf((float)d);  // AttentionScoreCalculationShader.cs:112
  const uint32_t group = qH / kvH;
#pragma omp parallel for schedule(static)
  for (int64_t hh = 0; hh < (int64_t)qH; ++hh) {
    uint32_t h = (uint32_t)hh;
    uint32_t g = h / group;
    std::vector<float> w(seq);
    for (uint32_t t = 0; t < seq; ++t) {
      const float* kr = kc + (uint64_t)t * kvDim + g * d;
      if (mode == 0) {
        float dot = 0.0f;
        for (uint32_t i = 0; i < d; ++i) dot += q[h * d + i] * kr[i];
        w[t] = dot * scale;
      } else {
        double dot = 0.0;
        for (uint32_t i = 0; i < d; ++i) dot += (double)q[h * d + i] * (double)kr[i];
        w[t] = (float)dot * scale;
      }
    }
    float mx = -1.0e38f;
    for (uint32_t t = 0; t < seq; ++t) mx = fmaxf(mx, w[t]);
    float inv;
    if (mode == 0) {
      float sum = 0.0f;
      for (uint32_t t = 0; t < seq; ++t) {
        float sc = w[t] - mx;
        sc = sc < -80.0f ? -80.0f : (sc > 80.0f ? 80.0f : sc);
        float e = expf(sc);
        w[t] = e;
        sum += e;
      }
      inv = sum > eps ? 1.0f / sum : 0.0f;
    } else {
      double sum = 0.0;
      for (uint32_t t = 0; t < seq; ++t) {
        float sc = w[t] - mx;
        sc = sc < -80.0f ? -80.0f : (sc > 80.0f ? 80.0f : sc);
        float e = expf(sc);
        w[t] = e;
        sum += (double)e;
      }
      inv = (float)sum > eps ? (float)(1.0 / sum) : 0.0f;
    }
    for (uint32_t t = 0; t < seq; ++t) w[t] = w[t] * inv;
    for (uint32_t i = 0; i < d; ++i) {
      if (mode == 0) {
        float acc = 0.0f;
        for (uint32_t t = 0; t < seq; ++t) acc += w[t] * vc[(uint64_t)t * kvDim + g * d + i];
        out[h * d + i] = acc;
      } else {
        double acc = 0.0;
        for (uint32_t t = 0; t < seq; ++t) acc += (double)w[t] * (double)vc[(uint64_t)t * kvDim + g * d + i];
        out[h * d + i] = (float)acc;
      }
    }
  }
}

// NFAI.Vulkan.Shaders/SiLUShader.cs:112-127 then ElementWiseMultiplicationShader.cs:127-138 with
// A = up, B = silu(gate) (TransformerBlock.cs:102,107): h = up * (gate * (1/(1+exp(-gate)))).
void silu_mul(const float* gate, const float* up, uint32_t F, float* h) {
  for (uint32_t j = 0; j < F; ++j) {
    float x = gate[j];
    float sig = 1.0f / (1.0f + expf(-x));
    float silu = x * sig;
    h[j] = up[j] * silu;
  }
}

Tensor* find_tensor(Model* m, const std::string& name) {
  if (name == "token_embd.weight") return &m->embd;
  if (name == "output_norm.weight") return &m->out_norm;
  if (name == "output.weight") return &m->out_head;
  if (name.rfind("blk.", 0) == 0) {
    size_t dot = name.find('.', 4);
    if (dot == std::string::npos) return nullptr;
    long li = strtol(name.substr(4, dot - 4).c_str(), nullptr, 10);
    if (li < 0 || li >= (long)m->layers.size()) return nullptr;
    Layer& L = m->layers[li];
    std::string rest = name.substr(dot + 1);
    if (rest == "attn_norm.weight") return &L.attn_norm;
    if (rest == "attn_q.weight") return &L.wq;
    if (rest == "attn_k.weight") return &L.wk;
    if (rest == "attn_v.weight") return &L.wv;
    if (rest == "attn_output.weight") return &L.wo;
    if (rest == "ffn_norm.weight") return &L.ffn_norm;
    if (rest == "ffn_gate.weight") return &L.wgate;
    if (rest == "ffn_up.weight") return &L.wup;
    if (rest == "ffn_down.weight") return &L.wdown;
  }
  return nullptr;
}

}  // namespace

extern "C" {

void* orc_create(const orc_hparams* hp) {
  if (!hp || hp->H == 0 || hp->L == 0 || hp->qH == 0 || hp->kvH == 0 || hp->d == 0 || hp->qH % hp->kvH != 0 ||
      hp->ctx == 0 || hp->V == 0 || hp->F == 0)
    return nullptr;
  Model* m = new Model();
  m->hp = *hp;
  m->layers.resize(hp->L);
  uint64_t kvDim = (uint64_t)hp->kvH * hp->d;
  m->kc.assign((uint64_t)hp->L * hp->ctx * kvDim, 0.0f);
  m->vc.assign((uint64_t)hp->L * hp->ctx * kvDim, 0.0f);
  rope_table(hp->ropeDim, hp->rope_theta, m->rope_f);
  m->hidden_taps.assign((uint64_t)hp->L * hp->H, 0.0f);
  m->last_q.assign((uint64_t)hp->L * hp->qH * hp->d, 0.0f);
  m->last_attn.assign((uint64_t)hp->L * hp->qH * hp->d, 0.0f);
  return m;
}

void orc_destroy(void* h) { delete (Model*)h; }

const char* orc_last_error(void* h) { return ((Model*)h)->err.c_str(); }

// dtype: 0 = float32, 1 = float16 (raw binary16 bits). The data is copied.
int orc_set_tensor(void* h, const char* name, int dtype, const void* data, uint64_t count) {
  Model* m = (Model*)h;
  Tensor* t = find_tensor(m, name);
  if (!t) { m->err = std::string("unknown tensor ") + name; return 1; }
  if (dtype != 0 && dtype != 1) { m->err = "bad dtype"; return 1; }
  t->dtype = dtype;
  t->count = count;
  if (dtype == 0) {
    t->f32.assign((const float*)data, (const float*)data + count);
    t->f16.clear();
  } else {
    t->f16.assign((const uint16_t*)data, (const uint16_t*)data + count);
    t->f32.clear();
  }
  return 0;
}

void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_reset(void* h) { ((Model*)h)->pos = 0; }
uint32_t orc_position(void* h) { return ((Model*)h)->pos; }
void orc_set_mode(void* h, int mode) { ((Model*)h)->hp.mode = mode; }

// Lowest index among the maxima: values.ToList().IndexOf(values.Max())
// (NFAI.Models.Llama3/SamplingUtils.cs:55-56).
uint32_t orc_argmax(const float* v, uint64_t n) {
  uint64_t best = 0;
  for (uint64_t i = 1; i < n; ++i)
    if (v[i] > v[best]) best = i;
  return (uint32_t)best;
}

// One token through the whole model at the current position; logits (V floats) may be null.
// Schedule and host-side residual adds: NFAI.Vulkan.Shaders/TransformerBlock.cs:127-184;
// model wiring (embed -> blocks -> output norm -> head bound to the embedding matrix):
// NFAI.Models.Llama3/LlamaModel.cs:43-67 and the per-token loop at :103-126, :134-173.
int orc_decode(void* h, uint32_t token, float* logits) {
  Model* m = (Model*)h;
  const orc_hparams& hp = m->hp;
  const int mode = hp.mode;
  if (m->pos >= hp.ctx) { m->err = "context full"; return 2; }
  if (token >= hp.V) { m->err = "token out of range"; return 1; }
  if (!m->embd.present() || !m->out_norm.present()) { m->err = "missing tensors"; return 3; }
  const uint32_t H = hp.H, d = hp.d, qDim = hp.qH * d, kvDim = hp.kvH * d, F = hp.F, p = m->pos;
  std::vector<float> x(H), a(H), q(qDim), o(qDim), t(H), up(F), gate(F), hbuf(F);
  // NFAI.Vulkan.Shaders/TokenEmbedShader.cs:139-158: out[d] = E[H*tok + d]
  for (uint32_t i = 0; i < H; ++i) x[i] = m->embd.at((uint64_t)H * token + i);
  for (uint32_t l = 0; l < hp.L; ++l) {
    Layer& L = m->layers[l];
    if (!L.wq.present() || !L.wk.present() || !L.wv.present() || !L.wo.present() || !L.wgate.present() ||
        !L.wup.present() || !L.wdown.present() || !L.attn_norm.present() || !L.ffn_norm.present()) {
      m->err = "missing layer tensors";
      return 3;
    }
    float* kcl = m->kc.data() + (uint64_t)l * hp.ctx * kvDim;
    float* vcl = m->vc.data() + (uint64_t)l * hp.ctx * kvDim;
    rmsnorm(x.data(), L.attn_norm, H, hp.eps, a.data(), mode);
    matvec(a.data(), L.wq, H, qDim, q.data(), mode);
    // K and V rows are written straight into the cache at row p (MatrixMultiplyShader.cs:286-287)
    matvec(a.data(), L.wk, H, kvDim, kcl + (uint64_t)p * kvDim, mode);
    matvec(a.data(), L.wv, H, kvDim, vcl + (uint64_t)p * kvDim, mode);
    rope(q.data(), hp.qH, d, hp.ropeDim, m->rope_f.data(), p);
    rope(kcl + (uint64_t)p * kvDim, hp.kvH, d, hp.ropeDim, m->rope_f.data(), p);  // in the cache, TransformerBlock.cs:71-74
    memcpy(m->last_q.data() + (uint64_t)l * qDim, q.data(), qDim * sizeof(float));
    attention(q.data(), kcl, vcl, p + 1, hp.qH, hp.kvH, d, hp.eps, o.data(), mode);
    memcpy(m->last_attn.data() + (uint64_t)l * qDim, o.data(), qDim * sizeof(float));
    matvec(o.data(), L.wo, qDim, H, t.data(), mode);
    for (uint32_t i = 0; i < H; ++i) x[i] = x[i] + t[i];  // TransformerBlock.cs:153-158
    rmsnorm(x.data(), L.ffn_norm, H, hp.eps, a.data(), mode);
    matvec(a.data(), L.wup, H, F, up.data(), mode);
    matvec(a.data(), L.wgate, H, F, gate.data(), mode);
    silu_mul(gate.data(), up.data(), F, hbuf.data());
    matvec(hbuf.data(), L.wdown, F, H, t.data(), mode);
    for (uint32_t i = 0; i < H; ++i) x[i] = x[i] + t[i];  // TransformerBlock.cs:176-180
    memcpy(m->hidden_taps.data() + (uint64_t)l * H, x.data(), H * sizeof(float));
  }
  m->pos = p + 1;
  if (logits) {
    rmsnorm(x.data(), m->out_norm, H, hp.eps, a.data(), mode);
    const Tensor& head = m->out_head.present() ? m->out_head : m->embd;
    matvec(a.data(), head, H, hp.V, logits, mode);
  }
  return 0;
}

// Debug taps for the parity tests.
int orc_read_kv(void* h, uint32_t layer, uint32_t pos, float* k, float* v) {
  Model* m = (Model*)h;
  const orc_hparams& hp = m->hp;
  if (layer >= hp.L || pos >= hp.ctx) return 1;
  uint64_t kvDim = (uint64_t)hp.kvH * hp.d;
  uint64_t off = ((uint64_t)layer * hp.ctx + pos) * kvDim;
  if (k) memcpy(k, m->kc.data() + off, kvDim * sizeof(float));
  if (v) memcpy(v, m->vc.data() + off, kvDim * sizeof(float));
  return 0;
}

int orc_write_kv(void* h, uint32_t layer, uint32_t pos, const float* k, const float* v) {
  Model* m = (Model*)h;
  const orc_hparams& hp = m->hp;
  if (layer >= hp.L || pos >= hp.ctx) return 1;
  uint64_t kvDim = (uint64_t)hp.kvH * hp.d;
  uint64_t off = ((uint64_t)layer * hp.ctx + pos) * kvDim;
  if (k) memcpy(m->kc.data() + off, k, kvDim * sizeof(float));
  if (v) memcpy(m->vc.data() + off, v, kvDim * sizeof(float));
  return 0;
}

void orc_set_position(void* h, uint32_t pos) { ((Model*)h)->pos = pos; }

int orc_read_hidden(void* h, uint32_t layer, float* out) {
  Model* m = (Model*)h;
  if (layer >= m->hp.L) return 1;
  memcpy(out, m->hidden_taps.data() + (uint64_t)layer * m->hp.H, m->hp.H * sizeof(float));
  return 0;
}

int orc_read_attn(void* h, uint32_t layer, float* q_rot, float* attn_out) {
  Model* m = (Model*)h;
  if (layer >= m->hp.L) return 1;
  uint64_t qDim = (uint64_t)m->hp.qH * m->hp.d;
  if (q_rot) memcpy(q_rot, m->last_q.data() + layer * qDim, qDim * sizeof(float));
  if (attn_out) memcpy(attn_out, m->last_attn.data() + layer * qDim, qDim * sizeof(float));
  return 0;
}

// ---- stand-alone operators, for kernel-level parity tests ------------------------------------------------

void orc_op_half_to_float(const uint16_t* in, float* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = half_to_float(in[i]);
}

void orc_op_rmsnorm(const float* x, const float* g, uint32_t H, float eps, float* y, int mode) {
  Tensor t;
  t.dtype = 0;
  t.f32.assign(g, g + H);
  rmsnorm(x, t, H, eps, y, mode);
}

void orc_op_matvec(const float* x, const void* W, int dtype, uint64_t K, uint64_t N, float* y, int mode) {
  if (dtype == 0) {
    const float* p = (const float*)W;
    matvec_rows(x, [p](uint64_t i) { return p[i]; }, K, N, y, mode);
  } else {
    const uint16_t* p = (const uint16_t*)W;
    matvec_rows(x, [p](uint64_t i) { return half_to_float(p[i]); }, K, N, y, mode);
  }
}

void orc_op_rope(float* v, uint32_t heads, uint32_t d, uint32_t ropeDim, float theta_base, uint32_t pos) {
  std::vector<float> f;
  rope_table(ropeDim, theta_base, f);
  rope(v, heads, d, ropeDim, f.data(), pos);
}

void orc_op_rope_table(uint32_t ropeDim, float theta_base, float* out) {
  std::vector<float> f;
  rope_table(ropeDim, theta_base, f);
  memcpy(out, f.data(), f.size() * sizeof(float));
}

void orc_op_attention(const float* q, const float* kc, const float* vc, uint32_t seq, uint32_t qH, uint32_t kvH,
                      uint32_t d, float eps, float* out, int mode) {
  attention(q, kc, vc, seq, qH, kvH, d, eps, out, mode);
}

void orc_op_silu_mul(const float* gate, const float* up, uint32_t F, float* h) { silu_mul(gate, up, F, h); }

}  // extern "C"

// ---- sampling ------------------------------------------------------------------------------------------------
// Temperature / top-k / top-p sampling exactly as NFAI.Models.Llama3/SamplingUtils.cs:5-33, with the uniform
// random number passed in (the reference draws it from Random.Shared): scaled = logit / T; probabilities by
// Softmax (:35-41: max, MathF.Exp(l - max), LINQ Sum = double accumulation returned as float, e / sum); stable sort
// by probability descending; the first top_k; accumulate until the cumulative probability reaches top_p;
// renormalise (LINQ Sum again); return the first index whose running sum exceeds u, else the last one.
extern "C" uint32_t orc_sample_top_p(const float* logits, uint64_t V, float temperature, float top_p, int top_k, float u) {
  std::vector<float> scaled(V);
  for (uint64_t i = 0; i < V; ++i) scaled[i] = logits[i] / temperature;
  float mx = scaled[0];
  for (uint64_t i = 1; i < V; ++i) mx = scaled[i] > mx ? scaled[i] : mx;
  std::vector<float> e(V);
  double sum = 0.0;
  for (uint64_t i = 0; i < V; ++i) {
    e[i] = expf(scaled[i] - mx);
    sum += (double)e[i];
  }
  const float sumf = (float)sum;
  std::vector<uint32_t> order(V);
  for (uint64_t i = 0; i < V; ++i) order[i] = (uint32_t)i;
  std::vector<float> prob(V);
  for (uint64_t i = 0; i < V; ++i) prob[i] = e[i] / sumf;
  // OrderByDescending is a stable sort: equal probabilities keep their index order
  std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return prob[a] > prob[b]; });
  const uint64_t k = (uint64_t)top_k < V ? (uint64_t)top_k : V;
  std::vector<uint32_t> idx;
  std::vector<float> pr;
  float cumulative = 0.f;
  for (uint64_t i = 0; i < k; ++i) {
    cumulative += prob[order[i]];
    idx.push_back(order[i]);
    pr.push_back(prob[order[i]]);
    if (cumulative >= top_p) break;
  }
  double tot = 0.0;
  for (float p : pr) tot += (double)p;
  const float total = (float)tot;
  float running = 0.f;
  for (size_t i = 0; i < pr.size(); ++i) {
    running += pr[i] / total;
    if (u < running) return idx[i];
  }
  return idx.back();
}

// ---- byte-pair merge loop of the reference tokenizer, literally (NFAI.Models.Llama3/Tokenizer.cs:130-166) -----
// For every adjacent pair of parts the whole merges list is scanned from the front until an entry equals the pair;
// the pair with the lowest entry index wins (the leftmost among equals), one merge is applied, and the scan starts
// over. parts / merges arrive as concatenated bytes with offset arrays (n + 1 entries; merges as 2 m + 1: left_0,
// right_0, left_1, ...). Writes the offsets of the merged parts (the bytes themselves do not move) and returns their
// number. Used to time the reference's algorithm in compiled code and to cross-check the Python restatement.
extern "C" uint32_t orc_bpe_merge_scan(const uint8_t* part_bytes, const uint32_t* part_off, uint32_t n_parts,
                                       const uint8_t* merge_bytes, const uint64_t* merge_off, uint32_t n_merges,
                                       uint32_t* out_off) {
  std::vector<std::pair<uint32_t, uint32_t>> parts;  // [begin, end) into part_bytes; merged parts stay contiguous
  for (uint32_t i = 0; i < n_parts; ++i) parts.push_back({part_off[i], part_off[i + 1]});
  auto equals = [&](const std::pair<uint32_t, uint32_t>& p, uint64_t mb, uint64_t me) {
    return (uint64_t)(p.second - p.first) == me - mb && memcmp(part_bytes + p.first, merge_bytes + mb, me - mb) == 0;
  };
  while (true) {
    long best_merge = -1, best_first = -1;
    for (size_t j = 0; j + 1 < parts.size(); ++j) {
      for (uint32_t k = 0; k < n_merges; ++k) {
        if (equals(parts[j], merge_off[2 * k], merge_off[2 * k + 1]) && equals(parts[j + 1], merge_off[2 * k + 1], merge_off[2 * k + 2])) {
          if (best_merge == -1 || (long)k < best_merge) {
            best_merge = (long)k;
            best_first = (long)j;
          }
          break;
        }
      }
    }
    if (best_merge == -1) break;
    parts[best_first].second = parts[best_first + 1].second;
    parts.erase(parts.begin() + best_first + 1);
  }
  for (size_t i = 0; i < parts.size(); ++i) out_off[i] = parts[i].first;
  out_off[parts.size()] = parts.empty() ? 0 : parts.back().second;
  return (uint32_t)parts.size();
}
