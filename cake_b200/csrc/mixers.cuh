// mixers.cuh — launch interface of the sequence mixers and the routed feed-forward of mixer-list blocks
// (cake_b200_block_load_mixer): latent attention (keys and values expanded from a cached low-rank latent), gated linear
// recurrences (a fixed decay per head, or input-dependent decays of a state-space layer), short causal convolutions,
// grouped unit norms with gates, and a mixture of experts with identity experts.  The kernels live in mixers.cu, a
// translation unit of its own; the entry points below take plain device pointers and a stream, so that any block
// structure can combine them.  Every function returns a cudaError_t cast to int and adds its launches to *launches.
//
// Nothing here follows a reference file: the reference has none of these layers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cake {
namespace mx {

// dtype codes are those of include/cake_b200.h (0 bf16, 1 f16, 2 f32): the type D of projections, caches and weights.
// Scores, softmax, norms, recurrent state, decays, routers and residual sums are fp32 whatever D is.

// ---- latent attention ------------------------------------------------------------------------------------------------
// Row m = (b, t) of a step of S tokens per batch row that starts at absolute position pos0.
struct LatentPrep {
  const void *proj;      // [M, ld] D: per head [dim | rot] query entries from column 0, then [rank | rot] at column kv_col
  int ld, kv_col;
  const void *norm_w;    // [rank] D
  const float *cos_t, *sin_t;  // [positions, rope_dims / 2]
  int rope_dims;         // <= rot: leading entries of the rotated part that are rotated (pairs i, i + rope_dims / 2)
  void *cache;           // [B, cap, rank + rot] D: the normed latent and the rotated shared key part
  void *cache_t;         // nullptr, or [B, rank, cap_t] D: the latent once more with the positions innermost (the second
  int cap_t;             // operand of the weights-times-latent product when it runs as a plain matrix product)
  void *qa;              // [M, heads, rank + rot] D: the rotated query part lands in columns rank..; columns 0..rank-1 are
                         // filled afterwards by the product of the unrotated query with the key expansion
  int B, S, heads, dim, rot, rank, cap, pos0;
  float eps;
};
int latent_prep(cudaStream_t, int dtype, const LatentPrep &, uint64_t *launches);

// softmax((qa . row_j) * scale over j <= position) weighted sum of the first `rank` columns of the cached rows
struct LatentAttn {
  const void *qa;        // [M, heads, rank + rot] D
  const void *cache;     // [B, cap, rank + rot] D
  void *lat;             // [M, heads, rank] D
  int B, S, heads, rank, rot, cap, pos0;
  float scale;
  // steps of a few rows: the keys of a (row, head) are split over nsplit CTAs whose partial (max, sum, weighted latent)
  // land in part [M * heads, nsplit, rank + 2] fp32 and are merged by a second kernel; nsplit <= 1: one warp per (row, head)
  float *part = nullptr;
  int nsplit = 0;
};
int latent_attention(cudaStream_t, int dtype, const LatentAttn &, uint64_t *launches);

// The same attention as matrix products for long portions in 16-bit D: scores [rows, kp] fp32 (rows = (t, head) pairs of `n_tok`
// tokens starting at step offset t0, kp keys padded to the product's tile) -> masked, scaled softmax -> the weights as
// w_hi + w_lo in D, [rows, 2 * kp]: hi in columns [0, kp), lo in [kp, 2 kp), zeros where row t sees no key.
struct LatentSoftmax {
  const float *scores;
  void *w;
  int n_tok, heads, kp, pos_first;   // pos_first: absolute position of the block's first token (it sees keys 0..pos_first)
  float scale;
};
int latent_softmax(cudaStream_t, int dtype, const LatentSoftmax &, uint64_t *launches);

// ---- batched small products: C[z][m, n] = sum_k A[z][m, k] * W[z][n, k]  (w_kn: W[z][k, n]) -------------------------------
struct HeadGemm {
  const void *A, *W;
  void *C;               // D
  int M, N, K, Z;
  long a_zs, w_zs, c_zs; // element offsets per z
  int lda, ldw, ldc;
  int w_kn;              // 1: W[z] is stored [K, N] row-major
};
int head_gemm(cudaStream_t, int dtype, const HeadGemm &, uint64_t *launches);

// out[z][c][r] = in[z][r][c] for Z matrices of [rows, cols] in D (weight layouts for the tensor-core products, at load)
int transpose_batched(cudaStream_t, int dtype, const void *in, void *out, int Z, int rows, int cols, uint64_t *launches);

// ---- gated linear recurrence -----------------------------------------------------------------------------------------
//   S_t = a_t S_{t-1} + b_t k_t v_t^T   (S: [dk, dv] fp32 per batch row and head),   o_t = S_t^T q_t + skip_h v_t
// fixed decay:      a_t = decay[h], b_t = kscale           (dt == nullptr)
// state space:      d = softplus(dt[m, h] + dt_bias[h]),  a_t = exp(-exp(a_log[h]) d),  b_t = d
// q and k of head h are read at column (h / group_div) * dk of their rows; with a rotation table the first rope_dims
// entries of q and k are rotated in fp32 on the way in.  The state is read unless pos0 == 0 and written back at the end.
struct Recurrence {
  const void *q, *k, *v; // D
  int ldq, ldk, ldv;
  int group_div;
  const void *dt;        // D [M, lddt] or nullptr
  int lddt;
  const void *dt_bias, *a_log, *skip;  // D [heads]; skip may be nullptr
  const float *decay;    // [heads] fp32
  float kscale;
  const float *cos_t, *sin_t;
  int rope_dims;
  float *state;          // [B, heads, dk, dv]
  float *o;              // [M, heads * dv] fp32
  int B, S, heads, dk, dv, pos0;
};
int recurrence(cudaStream_t, int dtype, const Recurrence &, uint64_t *launches);

// ---- short causal convolution per channel + silu -----------------------------------------------------------------------
struct ShortConv {
  const void *in;        // [M, ld] D, channels from column col0
  int ld, col0;
  const void *w, *bias;  // [channels, taps] (last tap = current token), [channels] D
  void *hist;            // [B, taps - 1, channels] D: the inputs before the step; updated to the step's last ones
  void *out;             // [M, channels] D
  int B, S, channels, taps, pos0;
};
int short_conv(cudaStream_t, int dtype, const ShortConv &, uint64_t *launches);

// ---- unit norm over equal parts of a row, with a gate before or after ------------------------------------------------
//   val = o * (gate_first ? silu(gate) : 1);  out = val / rms(val over its part) * (w ? w : 1) * (gate_first ? 1 : silu(gate))
struct GateNorm {
  const float *o;        // [M, n] fp32
  const void *gate;      // [M, ldg] D from column 0
  int ldg;
  const void *w;         // [n] D or nullptr
  void *out;             // [M, n] D
  int M, n, parts, gate_first;
  float eps;
};
int gate_norm(cudaStream_t, int dtype, const GateNorm &, uint64_t *launches);

// ---- routed feed-forward ---------------------------------------------------------------------------------------------
// Router: z = Wr h (fp32, a matrix product done by the caller), s = softmax(z); the `top` largest s + correction are chosen; weights = s / (sum of chosen + 1e-20)
// * scale.  Experts [0, experts) are gated feed-forwards, [experts, experts + identity) return their input.
struct MoePlan {
  const float *logits;   // [M, ld] fp32: router logits in columns [0, experts + identity); with has_shared_gate the logit of the
  int ld;                // shared expert's gate in the next column (sigmoid of it -> sgate[m])
  const void *correction;// [experts + identity] D
  int has_shared_gate;
  int M, W, experts, identity, top;
  float scale;
  int *ids;              // [M, top]
  float *wts;            // [M, top]
  float *sgate;          // [M]
  // grouping of the (token, slot) pairs by expert: every expert's pairs start on a multiple of `tile` sorted rows
  int tile;
  int *counts;           // [experts + 1] scratch
  int *perm;             // [max_tiles * tile]: sorted row -> m * top + slot, or -1 (padding)
  int *pos_of;           // [M * top]: m * top + slot -> sorted row (pairs of identity experts: untouched)
  int *tile_expert;      // [max_tiles]: the expert of a block of `tile` sorted rows, or -1 (unused block)
  int max_tiles;
};
int moe_route(cudaStream_t, int dtype, const MoePlan &, uint64_t *launches);

// sorted[r] = h[perm[r] / top] (zeros for padding rows): the operand of a grouped product on the tensor cores
int moe_gather(cudaStream_t, int dtype, const void *h, const int *perm, void *sorted, int rows, int W, int top, uint64_t *launches);

// CUDA-core experts for every shape and D = float: act = f(Wg h) * (Wu h), then y[sorted row] = Wd act
struct MoeExperts {
  const void *h;         // [M, W] D
  const void *wgu;       // [experts, 2 * ff, W] D: row 2i = gate_i, row 2i + 1 = up_i
  const void *wd;        // [experts, W, ff] D
  void *act;             // [max_tiles * tile, ff] D scratch
  float *y;              // [max_tiles * tile, W] fp32: expert outputs in sorted order, not yet weighted
  int M, W, ff, top, act_kind;
  const int *perm, *tile_expert;
  int tile, max_tiles;
};
int moe_experts(cudaStream_t, int dtype, const MoeExperts &, uint64_t *launches);

// x_out[m] = x[m] + sum over slots of wts * (expert: y[pos_of[m * top + slot]]; identity: h[m]), slots in order
struct MoeCombine {
  const float *x;
  float *x_out;
  const void *h;         // [M, W] D
  const float *y, *wts;
  const int *ids, *pos_of;
  int M, W, top, experts;
};
int moe_combine(cudaStream_t, int dtype, const MoeCombine &, uint64_t *launches);

// ---- x[m] += (x0 ? x0[m] : 0) + vec   (fp32 stream; vec [W] in D) --------------------------------------------------------
int stream_inject(cudaStream_t, int dtype, float *x, const float *x0, const void *vec, int M, int W, uint64_t *launches);

}  // namespace mx
}  // namespace cake
