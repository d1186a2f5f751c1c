// Linear attention with a fixed decay per head (no softmax, no denominator), as a recurrence over a
// per-sequence state, and the normalisation and gate that follow it.
//
//   S_t = decay_h * S_{t-1} + k_t v_t^T        S: [D, Dv] per (sequence, head), float32, kept from step to step
//   o_t = S_t^T q_t
//
// q, k and v come out of one fused projection (a row holds q heads, k heads, v heads and the gate's columns).
// What the design does to them before the recurrence happens while a chunk of tokens is staged in shared
// memory: an activation (none or SiLU), the rotation of q and k (pairs (i, i + n_rot/2) of a head's first
// n_rot dims, angle from float32 tables), a scale on k.  All of it, the state and the sums are float32.
//
// The recurrence is independent for every column of v, so a CTA owns `cols` columns of one (sequence, head)
// and walks that sequence's tokens of the step in order.  Within a CTA a warp owns 4 columns; the 8 lanes of
// a column split D among them in blocks of 4 dims (lane r owns dims 4 (r + 8 i) + 0..3), update their part of
// S and add up q . S with three shuffles.  The order of every addition is fixed by (d, column) alone, and a
// token's update is the same arithmetic whether it arrives in a prompt, in a later portion of one or alone, so
// a position's result does not depend on how tokens were cut into steps or batched, to the last bit.
//
// Work per token and head is 3 D Dv float32 operations (a multiply for k v, one fused multiply-add for the
// state, one for the output), which is what the FMA units are for; the state is read and written once per
// step, which is what bounds a decode step.
#include "common.cuh"

#define LA_CHUNK 16          // tokens staged per round
#define LA_MAX_D 256

enum { LA_ACT_NONE = 0, LA_ACT_SILU = 1, LA_ACT_SIGMOID = 2 };

__device__ __forceinline__ float la_act(float x, int act) {
  if (act == LA_ACT_SILU) return x / (1.0f + expf(-x));
  if (act == LA_ACT_SIGMOID) return 1.0f / (1.0f + expf(-x));
  return x;
}

// value of column c of token row t: one tensor, or split partials added in order
template <typename TIN>
__device__ __forceinline__ float la_value(const TIN* row, int c, int n_split, size_t split_stride) {
  float v = to_f32(row[c]);
  for (int s = 1; s < n_split; ++s) v += to_f32(row[s * split_stride + c]);
  return v;
}

// DPT: dims of D per thread (a multiple of 4; 8 threads share a column, so D <= 8 DPT).
template <typename TIN, int DPT>
__global__ void __launch_bounds__(256)
decay_scan_kernel(const TIN* __restrict__ proj, int n_split, size_t split_stride, size_t row_stride,
                  int q_off, int k_off, int v_off, float* __restrict__ out, float* __restrict__ state,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_past,
                  const int* __restrict__ seq_slot, const float* __restrict__ decay,
                  const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_rot, int act,
                  float k_scale, int H, int D, int Dv, int cols) {
  extern __shared__ float la_smem[];
  const int Dp = (D + 3) & ~3;                    // staged rows are padded to a multiple of 4 dims
  float* qs = la_smem;                            // [LA_CHUNK][Dp]
  float* ks = qs + LA_CHUNK * Dp;                 // [LA_CHUNK][Dp]
  float* vs = ks + LA_CHUNK * Dp;                 // [LA_CHUNK][cols]
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * cols;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col = c0 + warp * 4 + (lane >> 3);    // this thread's column of v
  const int r = lane & 7;                         // its share of D
  const bool col_live = (warp * 4 + (lane >> 3)) < cols && col < Dv;
  const int t0 = seq_start[b], n_new = seq_start[b + 1] - t0, past = seq_past[b];
  const float g = decay[h];
  float* S = state + ((size_t)seq_slot[b] * H + h) * (size_t)D * Dv;
  const int half = n_rot >> 1;
  pdl_wait();

  float s_reg[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = 4 * (r + 8 * (i >> 2)) + (i & 3);
    s_reg[i] = (col_live && d < D) ? S[(size_t)d * Dv + col] : 0.f;
  }

  for (int base = 0; base < n_new; base += LA_CHUNK) {
    const int n_tok = (n_new - base) < LA_CHUNK ? (n_new - base) : LA_CHUNK;
    __syncthreads();                              // the chunk before has been consumed
    // stage q and k of the chunk: activation, rotation, scale
    for (int e = tid; e < n_tok * Dp; e += blockDim.x) {
      const int tt = e / Dp, d = e - tt * Dp;
      float qv = 0.f, kv = 0.f;
      if (d < D) {
        const TIN* row = proj + (size_t)(t0 + base + tt) * row_stride;
        const TIN* qrow = row + q_off + h * D;
        const TIN* krow = row + k_off + h * D;
        qv = la_act(la_value(qrow, d, n_split, split_stride), act);
        kv = la_act(la_value(krow, d, n_split, split_stride), act);
        if (d < n_rot) {
          const int pos = past + base + tt;
          const int i = d < half ? d : d - half;
          const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
          const int partner = d < half ? d + half : d - half;
          const float qp = la_act(la_value(qrow, partner, n_split, split_stride), act);
          const float kp = la_act(la_value(krow, partner, n_split, split_stride), act);
          // (u, v) -> (u cos - v sin, v cos + u sin) for the pair (i, i + half)
          qv = d < half ? qv * c - qp * s : qv * c + qp * s;
          kv = d < half ? kv * c - kp * s : kv * c + kp * s;
        }
        kv *= k_scale;
      }
      qs[e] = qv;
      ks[e] = kv;
    }
    for (int e = tid; e < n_tok * cols; e += blockDim.x) {
      const int tt = e / cols, c = e - tt * cols;
      float v = 0.f;
      if (c0 + c < Dv) {
        const TIN* vrow = proj + (size_t)(t0 + base + tt) * row_stride + v_off + h * Dv;
        v = la_act(la_value(vrow, c0 + c, n_split, split_stride), act);
      }
      vs[e] = v;
    }
    __syncthreads();
    for (int tt = 0; tt < n_tok; ++tt) {
      const float v = vs[tt * cols + warp * 4 + (lane >> 3)];
      const float* qrow = qs + tt * Dp;
      const float* krow = ks + tt * Dp;
      float acc = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; ++i4) {
        const int d = 4 * (r + 8 * i4);
        if (d < Dp) {
          const float4 k4 = *reinterpret_cast<const float4*>(krow + d);
          const float4 q4 = *reinterpret_cast<const float4*>(qrow + d);
          float* s4 = s_reg + 4 * i4;
          s4[0] = fmaf(g, s4[0], k4.x * v);
          s4[1] = fmaf(g, s4[1], k4.y * v);
          s4[2] = fmaf(g, s4[2], k4.z * v);
          s4[3] = fmaf(g, s4[3], k4.w * v);
          acc = fmaf(s4[0], q4.x, acc);
          acc = fmaf(s4[1], q4.y, acc);
          acc = fmaf(s4[2], q4.z, acc);
          acc = fmaf(s4[3], q4.w, acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (r == 0 && col_live) out[(size_t)(t0 + base + tt) * H * Dv + (size_t)h * Dv + col] = acc;
    }
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = 4 * (r + 8 * (i >> 2)) + (i & 3);
    if (col_live && d < D) S[(size_t)d * Dv + col] = s_reg[i];
  }
}

// proj: [T, row_stride] (or split partials of it); out: float32 [T, H*Dv]; state: float32 [slots, H, D, Dv].
LLMX_API int llmx_decay_scan(const void* proj, int in_dtype, int n_split, long long split_stride, long long row_stride,
                             int q_off, int k_off, int v_off, float* out, float* state, const int* seq_start,
                             const int* seq_past, const int* seq_slot, const float* decay, const float* cos_t,
                             const float* sin_t, int n_rot, int act, float k_scale, int n_seqs, int H, int D, int Dv,
                             int n_sm, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || D <= 0 || D > LA_MAX_D || Dv <= 0 || n_split < 1 || n_rot < 0 || n_rot > D || (n_rot & 1))
    return LLMX_REFUSED(1);
  if (n_rot > 0 && (!cos_t || !sin_t)) return LLMX_REFUSED(4);
  if (act != LA_ACT_NONE && act != LA_ACT_SILU) return LLMX_REFUSED(1);
  if (n_seqs > 65535 || H > 65535) return LLMX_REFUSED(3);
  // columns per CTA: as many as still give every SM a CTA or two (a CTA with more columns stages q and k fewer times)
  int cols = 32;
  while (cols > 8 && (long long)n_seqs * H * ((Dv + cols - 1) / cols) < 2LL * n_sm) cols >>= 1;
  while (cols > 4 && cols / 2 >= Dv) cols >>= 1;
  const int Dp = (D + 3) & ~3;
  dim3 grid((Dv + cols - 1) / cols, H, n_seqs), block(cols * 8);
  const size_t smem = (size_t)LA_CHUNK * (2 * Dp + cols) * sizeof(float);
#define GO(TIN, DPT)                                                                                               \
  launch_pdl(decay_scan_kernel<TIN, DPT>, grid, block, smem, stream, (const TIN*)proj, n_split, (size_t)split_stride, \
             (size_t)row_stride, q_off, k_off, v_off, out, state, seq_start, seq_past, seq_slot, decay, cos_t, sin_t, \
             n_rot, act, k_scale, H, D, Dv, cols)
#define BY_D(TIN)                  \
  do {                             \
    if (Dp <= 32) GO(TIN, 4);      \
    else if (Dp <= 64) GO(TIN, 8); \
    else if (Dp <= 128) GO(TIN, 16); \
    else GO(TIN, 32);              \
  } while (0)
  if (in_dtype == LLMX_F32) BY_D(float);
  else if (in_dtype == LLMX_BF16) BY_D(bf16);
  else return LLMX_REFUSED(2);
#undef BY_D
#undef GO
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// After the recurrence: y[t, j] = o[t, j] * r * gain[j] * act(gate[t, j]) with r = 1 / sqrt(mean(o^2) + eps), the
// mean taken over one head's Dv columns (per_head, usually without a gain) or over all H*Dv columns of the
// token.  One warp per (token, head), or one CTA per token.  float32 throughout; y in the activations' dtype.
// ---------------------------------------------------------------------------
template <typename TIN, typename TO>
__global__ void gated_norm_heads_kernel(const float* __restrict__ o, const TIN* __restrict__ proj, int n_split,
                                        size_t split_stride, size_t row_stride, int g_off,
                                        const float* __restrict__ gain, float eps, int gate_act,
                                        TO* __restrict__ y, int H, int Dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x, h = blockIdx.y * 4 + warp;
  if (h >= H) return;
  const float* orow = o + ((size_t)t * H + h) * Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) ss += orow[i] * orow[i];
  const float r = 1.0f / sqrtf(warp_sum(ss) / (float)Dv + eps);
  const TIN* grow = proj + (size_t)t * row_stride + g_off + h * Dv;
  for (int i = lane; i < Dv; i += 32) {
    float v = orow[i] * r;
    if (gain) v *= gain[h * Dv + i];
    y[((size_t)t * H + h) * Dv + i] = from_f32<TO>(v * la_act(la_value(grow, i, n_split, split_stride), gate_act));
  }
}

template <typename TIN, typename TO>
__global__ void __launch_bounds__(256)
gated_norm_row_kernel(const float* __restrict__ o, const TIN* __restrict__ proj, int n_split, size_t split_stride,
                      size_t row_stride, int g_off, const float* __restrict__ gain, float eps, int gate_act,
                      TO* __restrict__ y, int n) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* orow = o + (size_t)t * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += orow[i] * orow[i];
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
  const TIN* grow = proj + (size_t)t * row_stride + g_off;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = orow[i] * r;
    if (gain) v *= gain[i];
    y[(size_t)t * n + i] = from_f32<TO>(v * la_act(la_value(grow, i, n_split, split_stride), gate_act));
  }
}

// per_head != 0: the mean of squares is a head's; else the token's.  gain: float32 [H*Dv] or null.
LLMX_API int llmx_gated_norm(const float* o, const void* proj, int in_dtype, int n_split, long long split_stride,
                             long long row_stride, int g_off, const float* gain, float eps, int gate_act, int per_head,
                             void* y, int out_dtype, int n_tokens, int H, int Dv, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || Dv <= 0 || n_split < 1) return LLMX_REFUSED(1);
  if (gate_act != LA_ACT_SILU && gate_act != LA_ACT_SIGMOID && gate_act != LA_ACT_NONE) return LLMX_REFUSED(1);
#define GO(TIN, TO)                                                                                                  \
  do {                                                                                                               \
    if (per_head)                                                                                                    \
      launch_pdl(gated_norm_heads_kernel<TIN, TO>, dim3(n_tokens, (H + 3) / 4), dim3(128), 0, stream, o,             \
                 (const TIN*)proj, n_split, (size_t)split_stride, (size_t)row_stride, g_off, gain, eps, gate_act,    \
                 (TO*)y, H, Dv);                                                                                     \
    else                                                                                                             \
      launch_pdl(gated_norm_row_kernel<TIN, TO>, dim3(n_tokens), dim3(256), 0, stream, o, (const TIN*)proj, n_split, \
                 (size_t)split_stride, (size_t)row_stride, g_off, gain, eps, gate_act, (TO*)y, H * Dv);              \
  } while (0)
  const int key = in_dtype * 2 + out_dtype;
  switch (key) {
    case 0: GO(float, float); break;
    case 1: GO(float, bf16); break;
    case 2: GO(bf16, float); break;
    case 3: GO(bf16, bf16); break;
    default: return LLMX_REFUSED(2);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}
