// Plain C++ references of the kernels' formulas, on the host: one short loop nest per operation, no tiling,
// no vector types, no device code (the file goes through the same build as the kernels so that it is found
// and loaded the same way).  Each kernel of this folder is tested against the function of the same name
// here; the functions follow the reference's CPU kernels statement by statement and are what a reader
// should open first to learn what a kernel computes.
//
//   pr_embedding     rows of a table                         crates/sglang-srt/src/cpu_reference.rs:741-752
//   pr_add_rms_norm  x = residual + delta; x / sqrt(mean(x^2) + eps) * w   crates/sglang-kernel/src/cpu.rs:26-34
//   pr_linear        y[o] = sum_i x[i] W[o, i] (+ b[o])     crates/sglang-kernel/src/cpu.rs:73-108
//   pr_gated_mul     act(g) * u                              crates/sglang-kernel/src/cpu.rs:119-123
//   pr_rope          rotation of pairs by pos * inv_freq     crates/sglang-kernel/src/rotary.rs:216-236
//   pr_attention     causal grouped-query attention          crates/sglang-kernel/src/cpu.rs:475-517
//   pr_argmax, pr_sample   greedy and temperature sampling   crates/sglang-srt/src/model_executor.rs:483-599
//
// Inputs and outputs are 32-bit floats; sums are kept in 64 bits, so that the functions are an oracle for the
// 32-bit kernels as well as for the bfloat16 ones (the reference's CPU code sums in 32 bits, in index order).
#include <math.h>
#include <stddef.h>

extern "C" {

const char* srb_last_error() { return ""; }

// out[r, :] = table[ids[r], :]; returns the number of ids outside the table (their rows are left untouched)
int pr_embedding(const int* ids, const float* table, int rows, int width, int vocab, float* out) {
  int bad = 0;
  for (int r = 0; r < rows; ++r) {
    if (ids[r] < 0 || ids[r] >= vocab) {
      ++bad;
      continue;
    }
    for (int i = 0; i < width; ++i) out[(size_t)r * width + i] = table[(size_t)ids[r] * width + i];
  }
  return bad;
}

// x = residual (+ delta); residual_out = x (if given); out = x / sqrt(mean(x^2) + eps) * weight
void pr_add_rms_norm(const float* residual, const float* delta, const float* weight, float eps, int rows, int width,
                     float* residual_out, float* out) {
  for (int r = 0; r < rows; ++r) {
    double sum = 0.0;
    for (int i = 0; i < width; ++i) {
      const double x = (double)residual[(size_t)r * width + i] + (delta ? (double)delta[(size_t)r * width + i] : 0.0);
      sum += x * x;
    }
    const double inv = 1.0 / sqrt(sum / width + (double)eps);
    for (int i = 0; i < width; ++i) {
      const double x = (double)residual[(size_t)r * width + i] + (delta ? (double)delta[(size_t)r * width + i] : 0.0);
      if (residual_out) residual_out[(size_t)r * width + i] = (float)x;
      out[(size_t)r * width + i] = (float)(x * inv * (double)weight[i]);
    }
  }
}

// y[m, n] = x[m, k] w[n, k]^T (+ bias[n])
void pr_linear(const float* x, const float* w, const float* bias, int m, int n, int k, float* y) {
  for (int r = 0; r < m; ++r)
    for (int o = 0; o < n; ++o) {
      double sum = 0.0;
      for (int i = 0; i < k; ++i) sum += (double)x[(size_t)r * k + i] * (double)w[(size_t)o * k + i];
      y[(size_t)r * n + o] = (float)(sum + (bias ? (double)bias[o] : 0.0));
    }
}

// out[r, j] = act(gate_up[r, j]) * gate_up[r, inner + j]; activation 0: g / (1 + exp(-g)); 1: the tanh form of GELU
void pr_gated_mul(const float* gate_up, int rows, int inner, int activation, float* out) {
  for (int r = 0; r < rows; ++r)
    for (int j = 0; j < inner; ++j) {
      const double g = gate_up[(size_t)r * 2 * inner + j], u = gate_up[(size_t)r * 2 * inner + inner + j];
      const double act = activation == 1 ? 0.5 * g * (1.0 + tanh(0.7978845608028654 * (g + 0.044715 * g * g * g)))
                                         : g / (1.0 + exp(-g));
      out[(size_t)r * inner + j] = (float)(act * u);
    }
}

// x: [rows, heads, head_dim], rotated in place over the first rotary_dim values of every head; the angle of pair i of
// row r is float(positions[r]) * inv_freq[i], both 32-bit, as the kernels and the reference's host code have it;
// pairs are (i, i + rotary_dim / 2), or (2i, 2i + 1) when interleaved
void pr_rope(float* x, const int* positions, const float* inv_freq, int rows, int heads, int head_dim, int rotary_dim,
             int interleaved) {
  const int half = rotary_dim / 2;
  for (int r = 0; r < rows; ++r)
    for (int h = 0; h < heads; ++h) {
      float* v = x + ((size_t)r * heads + h) * head_dim;
      for (int i = 0; i < half; ++i) {
        const float angle = (float)positions[r] * inv_freq[i];
        const double cs = cos((double)angle), sn = sin((double)angle);
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        const double a = v[ia], b = v[ib];
        v[ia] = (float)(a * cs - b * sn);
        v[ib] = (float)(b * cs + a * sn);
      }
    }
}

// q: [rows, n_q, d], the queries of one request at positions first_position .. first_position + rows - 1;
// k, v: [first_position + rows, n_kv, d], every key and value of the request.  A row at position p sees keys
// max(0, p - window + 1) .. p (window 0: all of them).  out like q.
void pr_attention(const float* q, const float* k, const float* v, int rows, int first_position, int n_q, int n_kv, int d,
                  float scale, int window, float* out, double* scratch /* first_position + rows doubles */) {
  const int group = n_q / n_kv;
  for (int r = 0; r < rows; ++r) {
    const int pos = first_position + r;
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    for (int h = 0; h < n_q; ++h) {
      const int kv = h / group;
      const float* qv = q + ((size_t)r * n_q + h) * d;
      double top = -INFINITY;
      for (int t = lo; t <= pos; ++t) {
        double s = 0.0;
        for (int e = 0; e < d; ++e) s += (double)qv[e] * (double)k[((size_t)t * n_kv + kv) * d + e];
        scratch[t] = s * (double)scale;
        if (scratch[t] > top) top = scratch[t];
      }
      double total = 0.0;
      for (int t = lo; t <= pos; ++t) {
        scratch[t] = exp(scratch[t] - top);
        total += scratch[t];
      }
      for (int e = 0; e < d; ++e) {
        double sum = 0.0;
        for (int t = lo; t <= pos; ++t) sum += scratch[t] * (double)v[((size_t)t * n_kv + kv) * d + e];
        out[((size_t)r * n_q + h) * d + e] = (float)(sum / total);
      }
    }
  }
}

// the index of the largest logit, the lowest index among equals
int pr_argmax(const float* logits, int vocab) {
  int best = 0;
  for (int i = 1; i < vocab; ++i)
    if (logits[i] > logits[best]) best = i;
  return best;
}

// inverse-CDF sampling of softmax(logits / temperature) with the uniform number u in [0, 1), walking the vocabulary
// in index order
int pr_sample(const float* logits, int vocab, float temperature, float u) {
  double top = -INFINITY;
  for (int i = 0; i < vocab; ++i) top = fmax(top, (double)logits[i] / temperature);
  double total = 0.0;
  for (int i = 0; i < vocab; ++i) total += exp((double)logits[i] / temperature - top);
  double running = 0.0;
  const double target = (double)u * total;
  for (int i = 0; i < vocab; ++i) {
    running += exp((double)logits[i] / temperature - top);
    if (running > target) return i;
  }
  return vocab - 1;
}

}  // extern "C"
