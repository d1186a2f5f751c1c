// A short causal convolution over time on every channel of a fused q|k|v projection, followed by what the
// attention mixer does to its heads before it attends: rotation of q and k, mixing of the values with those
// of an earlier layer, the cache write of k and v.
//
//   y_p[c] = sum_j w[c][j] * u_(p - taps + 1 + j)[c],   j = 0..taps-1,   u = 0 before the sequence's start
//
// u of the positions before the step's first token comes from the sequence's state: the last taps-1 projected
// rows, float32 [slot][taps-1][C], oldest first (zero-filled when the slot gets its owner, which is also what
// positions before the start must read).  conv_state_update moves the state on by the step's tokens; it is a
// second kernel because the first one's CTAs still read the old state.
//
// Row layout of the projection: q heads (H of D), k heads (G of D), v heads (G of Dv); C = (H+G) D + G Dv.
// One warp per (token, head).  The convolved head is staged in shared memory so that a dim can read its
// rotation partner (i, i + n_rot/2).  Values: v_mix_mode 1 writes the head to v_first (float32 [T, G Dv]) as
// well; 2 replaces it by (1 - lambda) v + lambda v_first before the cache write.  All arithmetic is float32
// in a fixed order (taps oldest first, partials in order).
#include "common.cuh"

#define SC_WARPS 4
#define SC_MAX_TAPS 16

template <typename TIN>
__device__ __forceinline__ float sc_value(const TIN* p, int n_split, size_t split_stride) {
  float v = to_f32(p[0]);
  for (int s = 1; s < n_split; ++s) v += to_f32(p[(size_t)s * split_stride]);
  return v;
}

template <typename TIN, typename TA, typename TC>
__global__ void conv_rope_cache_kernel(const TIN* __restrict__ proj, int n_split, size_t split_stride,
                                       const float* __restrict__ state, const float* __restrict__ conv_w, int taps,
                                       TA* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                       const int* __restrict__ block_table, int table_width,
                                       const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                       const int* __restrict__ seq_start, const int* __restrict__ seq_past,
                                       const int* __restrict__ seq_slot, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int n_rot, float* __restrict__ v_first,
                                       const float* __restrict__ v_lambda, int v_mix_mode, int H, int G, int D, int Dv) {
  extern __shared__ float head_buf[];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int slot_h = blockIdx.y * SC_WARPS + warp;           // which head of the fused row
  if (slot_h >= H + 2 * G) return;
  const size_t C = (size_t)(H + G) * D + (size_t)G * Dv;
  const bool is_q = slot_h < H, is_k = !is_q && slot_h < H + G;
  const int hd = (is_q || is_k) ? D : Dv;
  const size_t c0 = (is_q || is_k) ? (size_t)slot_h * D : (size_t)(H + G) * D + (size_t)(slot_h - H - G) * Dv;
  const int b = token_seq[t], pos = token_pos[t];
  const int p0 = seq_past[b], row0 = seq_start[b];
  const float* st = taps > 1 ? state + (size_t)seq_slot[b] * (taps - 1) * C : nullptr;
  const int page = is_q ? 0 : block_table[(size_t)b * table_width + pos / LLMX_PAGE];
  const float lam = v_mix_mode == 2 ? v_lambda[0] : 0.f;
  float* buf = head_buf + warp * max(D, Dv);
  pdl_wait();
  for (int i = lane; i < hd; i += 32) {
    const size_t c = c0 + i;
    float y;
    if (taps > 0) {
      y = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int pp = pos - taps + 1 + j;
        float u = 0.f;
        if (pp >= p0) u = sc_value(proj + (size_t)(row0 + pp - p0) * C + c, n_split, split_stride);
        else if (pp >= 0) u = st[(size_t)(pp - (p0 - (taps - 1))) * C + c];
        y = fmaf(conv_w[c * taps + j], u, y);
      }
    } else {
      y = sc_value(proj + (size_t)t * C + c, n_split, split_stride);
    }
    buf[i] = y;
  }
  __syncwarp();
  if (is_q || is_k) {
    const int half = n_rot >> 1;
    const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sv = sin_t ? sin_t + (size_t)pos * half : nullptr;
    TA* qrow = is_q ? q_out + (size_t)t * H * D + (size_t)slot_h * D : nullptr;
    TC* krow = is_k ? k_cache + cache_row_offset(page, slot_h - H, pos % LLMX_PAGE, G, D) : nullptr;
    for (int i = lane; i < D; i += 32) {
      float v = buf[i];
      if (i < half) v = buf[i] * c[i] - buf[i + half] * sv[i];
      else if (i < n_rot) v = buf[i] * c[i - half] + buf[i - half] * sv[i - half];
      if (is_q) qrow[i] = from_f32<TA>(v);
      else krow[i] = from_f32<TC>(v);
    }
  } else {
    const int g = slot_h - H - G;
    TC* vrow = v_cache + cache_row_offset(page, g, pos % LLMX_PAGE, G, Dv);
    float* first = v_mix_mode ? v_first + (size_t)t * G * Dv + (size_t)g * Dv : nullptr;
    for (int i = lane; i < Dv; i += 32) {
      float v = buf[i];
      if (v_mix_mode == 1) first[i] = v;
      else if (v_mix_mode == 2) v = (1.0f - lam) * v + lam * first[i];
      vrow[i] = from_f32<TC>(v);
    }
  }
}

// One thread per (sequence, channel): the state's rows become the projected rows of the last taps-1 positions
// after the step (old rows where the step brought fewer tokens than that).
template <typename TIN>
__global__ void conv_state_update_kernel(const TIN* __restrict__ proj, int n_split, size_t split_stride,
                                         float* __restrict__ state, int taps, const int* __restrict__ seq_start,
                                         const int* __restrict__ seq_slot, int n_seqs, size_t C) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C || b >= n_seqs) return;
  const int row0 = seq_start[b], n_new = seq_start[b + 1] - row0;
  const int keep = taps - 1;
  float* st = state + (size_t)seq_slot[b] * keep * C + c;
  float nv[SC_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < SC_MAX_TAPS; ++i) {
    if (i >= keep) break;
    const int j = n_new - keep + i;          // place among the step's tokens; negative: still an old row
    nv[i] = j >= 0 ? sc_value(proj + (size_t)(row0 + j) * C + c, n_split, split_stride) : st[(size_t)(i + n_new) * C];
  }
#pragma unroll
  for (int i = 0; i < SC_MAX_TAPS; ++i) {
    if (i >= keep) break;
    st[(size_t)i * C] = nv[i];
  }
}

// proj [T, C] or n_split float32 partials; conv_w float32 [C, taps] (taps 0: no convolution); state float32
// [slots, taps-1, C]; q_out [T, H*D]; cos/sin float32 [positions, n_rot/2]; v_first float32 [T, G*Dv] (v_mix_mode
// 1: written, 2: read with the weight *v_lambda).
LLMX_API int llmx_conv_rope_cache(const void* proj, int in_dtype, int n_split, long long split_stride, const float* state,
                                  const float* conv_w, int taps, void* q_out, int act_dtype, void* k_cache, void* v_cache,
                                  int cache_dtype, const int* block_table, int table_width, const int* token_seq,
                                  const int* token_pos, const int* seq_start, const int* seq_past, const int* seq_slot,
                                  const float* cos_t, const float* sin_t, int n_rot, float* v_first, const float* v_lambda,
                                  int v_mix_mode, int n_tokens, int H, int G, int D, int Dv, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || D <= 0 || Dv <= 0 || n_rot < 0 || n_rot > D || (n_rot & 1) || n_split < 1 || taps < 0 ||
      taps > SC_MAX_TAPS || v_mix_mode < 0 || v_mix_mode > 2)
    return LLMX_REFUSED(1);
  if ((n_rot > 0 && (!cos_t || !sin_t)) || (taps > 0 && !conv_w) || (taps > 1 && !state) || (v_mix_mode && !v_first) ||
      (v_mix_mode == 2 && !v_lambda))
    return LLMX_REFUSED(4);
  const int hd = D > Dv ? D : Dv;
  const size_t smem = (size_t)SC_WARPS * hd * sizeof(float);
  if (smem > 48 * 1024) return LLMX_REFUSED(3);
  dim3 grid(n_tokens, (H + 2 * G + SC_WARPS - 1) / SC_WARPS);
#define CASE(TIN, TA, TC)                                                                                            \
  launch_pdl(conv_rope_cache_kernel<TIN, TA, TC>, grid, dim3(SC_WARPS * 32), smem, stream, (const TIN*)proj, n_split, \
             (size_t)split_stride, state, conv_w, taps, (TA*)q_out, (TC*)k_cache, (TC*)v_cache, block_table,           \
             table_width, token_seq, token_pos, seq_start, seq_past, seq_slot, cos_t, sin_t, n_rot, v_first, v_lambda, \
             v_mix_mode, H, G, D, Dv)
  const int key = in_dtype * 4 + act_dtype * 2 + cache_dtype;
  switch (key) {
    case 0: CASE(float, float, float); break;
    case 1: CASE(float, float, bf16); break;
    case 2: CASE(float, bf16, float); break;
    case 3: CASE(float, bf16, bf16); break;
    case 6: CASE(bf16, bf16, float); break;
    case 7: CASE(bf16, bf16, bf16); break;
    default: return LLMX_REFUSED(2);
  }
#undef CASE
  return LLMX_LAUNCH_STATUS();
}

LLMX_API int llmx_conv_state_update(const void* proj, int in_dtype, int n_split, long long split_stride, float* state,
                                    int taps, const int* seq_start, const int* seq_slot, int n_seqs, long long C,
                                    cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return 0;
  if (taps > SC_MAX_TAPS || C <= 0 || n_split < 1 || n_seqs > 65535) return LLMX_REFUSED(1);
  dim3 grid((unsigned)((C + 127) / 128), n_seqs);
  if (in_dtype == LLMX_F32)
    launch_pdl(conv_state_update_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, n_split,
               (size_t)split_stride, state, taps, seq_start, seq_slot, n_seqs, (size_t)C);
  else if (in_dtype == LLMX_BF16)
    launch_pdl(conv_state_update_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)proj, n_split,
               (size_t)split_stride, state, taps, seq_start, seq_slot, n_seqs, (size_t)C);
  else
    return LLMX_REFUSED(2);
  return LLMX_LAUNCH_STATUS();
}
