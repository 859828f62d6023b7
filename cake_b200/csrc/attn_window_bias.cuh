// attn_window_bias.cuh — grouped-query attention with the score modifiers of the layer-list blocks (include/cake_b200.h,
// cake_b200_layer_spec), all of them parameters:
//
//   s_ij = (q_i . k_j) * scale
//   softcap > 0      s <- softcap * tanh(s / softcap)
//   r1, r2 non-null  s <- s - r1[h] * ln(1 + r2[h] * (i - j))           (a bias that grows with the distance, per query head)
//   window > 0       i sees j with 0 <= i - j < window; window == 0: every j <= i
//   p = softmax over the visible j (fp32);   out_i = sum_j p_ij v_j   with v == k when the values are the keys (vc == kc)
//   gate_col >= 0    out_i <- out_i * sigmoid(z_ih), z_ih = column gate_col + h of the projection row of token i
//
// Scores, bias, softmax and the weighted sum are fp32 whatever D is.  Keys are read only from the cache (the step's own
// keys are appended before the launch), so a position's result does not depend on how the prompt was cut into steps.
// Kernels:
//   attn_window_bias_kernel      one warp per (token, head), any head_dim <= 256 and any D (float included): a lane scores
//                                one key of a 32-key tile, the tile's keys are then accumulated dimension-parallel
//   attn_window_decode_kernel    one CTA per (batch row, head) for single-token steps: its warps split the window and merge
//                                their partial softmax states in shared memory
// Nothing here follows a reference file: the reference has none of these modifiers.
#pragma once
#include "common.cuh"
#include "f32_stream.cuh"

namespace cake {

struct WinAttn {
  const void *qkg;       // [B*S, ld] D: q of head h at columns [h*hd, (h+1)*hd); gate logits at gate_col + h
  const void *kc, *vc;   // [B, n_kv, cap, hd] D
  const void *r1, *r2;   // [heads] D or null
  void *y;               // [B*S, ldy] D: head h at columns [h*hd, (h+1)*hd)
  int B, S, heads, n_kv, hd, cap, pos0, ld, ldy, gate_col, window;
  float scale, softcap;
};
constexpr int WA_MAX_HD = 256;

// q (fp32, shared memory) . k (D, global), 16-byte loads when the row allows them
template <typename T> __device__ __forceinline__ float wa_dot(const float *q, const T *k, int hd);
template <> __device__ __forceinline__ float wa_dot<float>(const float *q, const float *k, int hd) {
  float s = 0.f;
  if ((hd & 3) == 0) {
    const float4 *k4 = reinterpret_cast<const float4 *>(k);
    for (int i = 0; i < hd / 4; i++) {
      const float4 v = k4[i];
      s = fmaf(q[4 * i], v.x, s); s = fmaf(q[4 * i + 1], v.y, s); s = fmaf(q[4 * i + 2], v.z, s); s = fmaf(q[4 * i + 3], v.w, s);
    }
  } else
    for (int i = 0; i < hd; i++) s = fmaf(q[i], k[i], s);
  return s;
}
template <typename T> __device__ __forceinline__ float wa_dot(const float *q, const T *k, int hd) {
  float s = 0.f;
  if ((hd & 7) == 0) {
    const uint4 *k4 = reinterpret_cast<const uint4 *>(k);
    for (int i = 0; i < hd / 8; i++) {
      float f[8];
      unpack8<T>(k4[i], f);
#pragma unroll
      for (int e = 0; e < 8; e++) s = fmaf(q[8 * i + e], f[e], s);
    }
  } else
    for (int i = 0; i < hd; i++) s = fmaf(q[i], DT<T>::to_f(k[i]), s);
  return s;
}

// the modified score of query position pi against key position pj (visible keys only)
__device__ __forceinline__ float wa_score(float dot, const WinAttn &p, float r1, float r2, bool biased, int pi, int pj) {
  float s = dot * p.scale;
  if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
  if (biased) s -= r1 * logf(1.0f + r2 * (float)(pi - pj));
  return s;
}

template <typename T>
__global__ void __launch_bounds__(128) attn_window_bias_kernel(const WinAttn p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float qs[4][WA_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * 4 + warp;
  if (item >= (long)p.B * p.S * p.heads) return;
  const int h = (int)(item % p.heads);
  const int t = (int)((item / p.heads) % p.S);
  const int b = (int)(item / ((long)p.heads * p.S));
  const int hd = p.hd, G = p.heads / p.n_kv;
  const T *qrow = reinterpret_cast<const T *>(p.qkg) + (size_t)(b * p.S + t) * p.ld;
  const T *kc = reinterpret_cast<const T *>(p.kc) + ((size_t)b * p.n_kv + h / G) * p.cap * hd;
  const T *vc = reinterpret_cast<const T *>(p.vc) + ((size_t)b * p.n_kv + h / G) * p.cap * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = DT<T>::to_f(qrow[h * hd + d]);
  __syncwarp();
  const bool biased = p.r1 != nullptr;
  const float r1 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r1)[h]) : 0.f;
  const float r2 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r2)[h]) : 0.f;
  const int pi = p.pos0 + t;
  const int lo = p.window > 0 ? max(0, pi - p.window + 1) : 0;
  constexpr int MAXD = WA_MAX_HD / 32;
  float acc[MAXD];
#pragma unroll
  for (int i = 0; i < MAXD; i++) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int j0 = lo; j0 <= pi; j0 += 32) {
    const int j = j0 + lane;
    const bool vis = j <= pi;
    float s = -INFINITY;
    if (vis) s = wa_score(wa_dot<T>(qs[warp], kc + (size_t)j * hd, hd), p, r1, r2, biased, pi, j);
    const float mn = fmaxf(m, warp_max(s));
    const float f = (m == -INFINITY) ? 0.f : expf(m - mn);
    const float e = vis ? expf(s - mn) : 0.f;
    l = l * f + warp_sum(e);
    m = mn;
#pragma unroll
    for (int i = 0; i < MAXD; i++) acc[i] *= f;
    const int cnt = min(32, pi - j0 + 1);
    for (int jj = 0; jj < cnt; jj++) {
      const float pj = __shfl_sync(0xffffffffu, e, jj);
      const T *vr = vc + (size_t)(j0 + jj) * hd;
#pragma unroll
      for (int i = 0; i < MAXD; i++) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, DT<T>::to_f(vr[d]), acc[i]);
      }
    }
  }
  float gate = 1.0f;
  if (p.gate_col >= 0) gate = 1.0f / (1.0f + expf(-DT<T>::to_f(qrow[p.gate_col + h])));
  const float inv = gate / l;
  T *yo = reinterpret_cast<T *>(p.y) + (size_t)(b * p.S + t) * p.ldy + h * hd;
#pragma unroll
  for (int i = 0; i < MAXD; i++) {
    const int d = lane + 32 * i;
    if (d < hd) yo[d] = DT<T>::from_f(acc[i] * inv);
  }
}

}  // namespace cake
