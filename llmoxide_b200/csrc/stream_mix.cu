// Several copies of the residual stream ("hyper-connections") and the norm that reads them.
//
// The stream is h [S][T][d], float32.  A sublayer reads u = sum_s read[s] h_s through an RMS norm; its result y
// joins the copies as h_r <- sum_s mix[s][r] h_s + write[r] y (every copy from the old ones; `write` already
// holds the layer's residual factor).  As with the single stream, the update that a sublayer owes is applied by
// the norm kernel of the NEXT sublayer, which then reads the new copies while they are in registers:
//
//   for row t (t = rows ? rows[r] : r), every column i:
//     x_s = h[s][t][i]
//     if update: y = sum_p delta[p][t][i] (partials in order); x'_r = sum_s mix[s][r] x_s + write[r] y;
//                h[r][t][i] = x'_r when write_h
//     u = sum_s read[s] x'_s            (read == nullptr: the plain sum of the copies)
//     out[r][i] = u / sqrt(mean_i(u^2) + eps) * gain[i]      (out == nullptr: only the update)
//
// Everything is float32 and every sum runs in an order fixed by (s, p, i) alone: a row's result does not depend
// on the batch.  One CTA per row; u is staged in shared memory between the two passes.
#include "common.cuh"

#define SM_MAX_STREAMS 8

template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
stream_mix_norm_kernel(float* __restrict__ h, size_t stream_stride, int S, const TD* __restrict__ delta, int n_split,
                       size_t split_stride, const float* __restrict__ mix, const float* __restrict__ write,
                       const float* __restrict__ read, const int* __restrict__ rows, const float* __restrict__ gain,
                       float eps, TO* __restrict__ out, int d, int write_h) {
  extern __shared__ float u_buf[];   // [d]
  __shared__ float red[32];
  __shared__ float w_mix[SM_MAX_STREAMS * SM_MAX_STREAMS], w_write[SM_MAX_STREAMS], w_read[SM_MAX_STREAMS];
  pdl_launch_dependents();
  // the connection weights and the row index are weights and step inputs: fetched ahead of the dependency wait
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  const bool update = mix != nullptr;
  if (threadIdx.x < S * S) w_mix[threadIdx.x] = update ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    w_write[threadIdx.x] = update ? write[threadIdx.x] : 0.f;
    w_read[threadIdx.x] = read ? read[threadIdx.x] : 1.0f;
  }
  __syncthreads();
  pdl_wait();
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x[SM_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < SM_MAX_STREAMS; ++s)
      if (s < S) x[s] = h[(size_t)s * stream_stride + (size_t)t * d + i];
    if (update) {
      float y = 0.f;
      if (delta) {
        const TD* p = delta + (size_t)t * d + i;
        for (int sp = 0; sp < n_split; ++sp) y += to_f32(p[(size_t)sp * split_stride]);
      }
      float nx[SM_MAX_STREAMS];
#pragma unroll
      for (int to = 0; to < SM_MAX_STREAMS; ++to) {
        if (to >= S) break;
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < SM_MAX_STREAMS; ++s)
          if (s < S) acc = fmaf(w_mix[s * S + to], x[s], acc);
        nx[to] = fmaf(w_write[to], y, acc);
      }
#pragma unroll
      for (int s = 0; s < SM_MAX_STREAMS; ++s)
        if (s < S) {
          x[s] = nx[s];
          if (write_h) h[(size_t)s * stream_stride + (size_t)t * d + i] = nx[s];
        }
    }
    if (out) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < SM_MAX_STREAMS; ++s)
        if (s < S) u = fmaf(w_read[s], x[s], u);
      u_buf[i] = u;
      ss += u * u;
    }
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float scale = 1.0f / sqrtf(total / (float)d + eps);
  TO* orow = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) orow[i] = from_f32<TO>((u_buf[i] * scale) * gain[i]);
}

// h float32 [S, T, d] (copy s at h + s * stream_stride).  delta: null, or n_split partials [T, d] (split_stride
// apart).  mix [S*S] (from, to) and write [S]: the update to apply first, or null for none.  read [S] or null
// (all ones).  rows: null or n_rows row indices.  out: null or [n_rows, d].
LLMX_API int llmx_stream_mix_norm(float* h, long long stream_stride, int S, const void* delta, int delta_dtype,
                                  int n_split, long long split_stride, const float* mix, const float* write,
                                  const float* read, const int* rows, int n_rows, const float* gain, float eps,
                                  void* out, int out_dtype, int d, int write_h, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (S <= 0 || S > SM_MAX_STREAMS || d <= 0 || n_split < 1) return LLMX_REFUSED(1);
  if ((mix == nullptr) != (write == nullptr) || (delta && !mix) || (out && !gain)) return LLMX_REFUSED(4);
  const size_t smem = out ? (size_t)d * sizeof(float) : 0;
  if (smem > 200 * 1024) return LLMX_REFUSED(3);
#define CASE(TD, TO)                                                                                              \
  do {                                                                                                            \
    if (smem > 48 * 1024)                                                                                         \
      cudaFuncSetAttribute(stream_mix_norm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_pdl(stream_mix_norm_kernel<TD, TO>, dim3(n_rows), dim3(256), smem, stream, h, (size_t)stream_stride, S, \
               (const TD*)delta, n_split, (size_t)split_stride, mix, write, read, rows, gain, eps, (TO*)out, d,    \
               write_h);                                                                                          \
  } while (0)
  if (delta_dtype == LLMX_F32 && out_dtype == LLMX_F32) CASE(float, float);
  else if (delta_dtype == LLMX_F32 && out_dtype == LLMX_BF16) CASE(float, bf16);
  else if (delta_dtype == LLMX_BF16 && out_dtype == LLMX_BF16) CASE(bf16, bf16);
  else if (delta_dtype == LLMX_BF16 && out_dtype == LLMX_F32) CASE(bf16, float);
  else return LLMX_REFUSED(2);
#undef CASE
  return LLMX_LAUNCH_STATUS();
}
