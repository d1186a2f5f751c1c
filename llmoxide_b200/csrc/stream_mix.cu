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
// on the batch.  One CTA per row, four columns per thread and load where the rows' alignment allows; u is staged
// in shared memory between the two passes.
#include "common.cuh"

#define SM_MAX_STREAMS 8

// Four columns at a time (d a multiple of 4: every row then starts on a 16-byte boundary), or one (VEC == 1).
template <int VEC> struct SmVec;
template <> struct SmVec<1> {
  float v[1];
};
template <> struct SmVec<4> {
  float v[4];
};
__device__ __forceinline__ void sm_load(const float* p, SmVec<1>& o) { o.v[0] = p[0]; }
__device__ __forceinline__ void sm_load(const bf16* p, SmVec<1>& o) { o.v[0] = __bfloat162float(p[0]); }
__device__ __forceinline__ void sm_load(const float* p, SmVec<4>& o) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  o.v[0] = x.x, o.v[1] = x.y, o.v[2] = x.z, o.v[3] = x.w;
}
__device__ __forceinline__ void sm_load(const bf16* p, SmVec<4>& o) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  o.v[0] = a.x, o.v[1] = a.y, o.v[2] = b.x, o.v[3] = b.y;
}
__device__ __forceinline__ void sm_store(float* p, const SmVec<1>& o) { p[0] = o.v[0]; }
__device__ __forceinline__ void sm_store(bf16* p, const SmVec<1>& o) { p[0] = __float2bfloat16_rn(o.v[0]); }
__device__ __forceinline__ void sm_store(float* p, const SmVec<4>& o) {
  *reinterpret_cast<float4*>(p) = make_float4(o.v[0], o.v[1], o.v[2], o.v[3]);
}
__device__ __forceinline__ void sm_store(bf16* p, const SmVec<4>& o) {
  __nv_bfloat162 a = __floats2bfloat162_rn(o.v[0], o.v[1]), b = __floats2bfloat162_rn(o.v[2], o.v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

#define SM_MAX_PARTS 4      // partials whose loads go out together with the copies' (more are added one by one)

// MAXS: the most copies this instance takes (its arrays live in registers: a kernel for eight copies that is
// handed four would hold twice the registers it needs and halve the CTAs per SM).
template <typename TD, typename TO, int VEC, int MAXS>
__global__ void __launch_bounds__(512)
stream_mix_norm_kernel(float* __restrict__ h, size_t stream_stride, int S, const TD* __restrict__ delta, int n_split,
                       size_t split_stride, const float* __restrict__ mix, const float* __restrict__ write,
                       const float* __restrict__ read, const int* __restrict__ rows, const float* __restrict__ gain,
                       float eps, TO* __restrict__ out, int d, int write_h, int n_tokens) {
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
  if (t < 0 || t >= n_tokens) {        // a row index that does not fit the stream: reported, nothing is touched
    if (threadIdx.x == 0) llmx_report(1);
    return;
  }
  // the connection weights in registers (one shared-memory read each, not one per column)
  // for up to four copies; more stay in shared memory, or the kernel would spill
  constexpr bool REGW = MAXS <= 4;
  constexpr int RW = REGW ? MAXS : 1;
  float r_mix[RW][RW], r_write[RW], r_read[RW];
#pragma unroll
  for (int s = 0; s < RW; ++s) {
    r_write[s] = s < S ? w_write[s] : 0.f;
    r_read[s] = s < S ? w_read[s] : 0.f;
#pragma unroll
    for (int to = 0; to < RW; ++to) r_mix[s][to] = (s < S && to < S) ? w_mix[s * S + to] : 0.f;
  }
  pdl_wait();
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < d; i += blockDim.x * VEC) {
    // every load of this thread's columns goes out before the first is used: the copies, then the partials
    SmVec<VEC> x[MAXS], part[SM_MAX_PARTS];
#pragma unroll
    for (int s = 0; s < MAXS; ++s)
      if (s < S) sm_load(h + (size_t)s * stream_stride + (size_t)t * d + i, x[s]);
    const TD* p = (update && delta) ? delta + (size_t)t * d + i : nullptr;
    if (p) {
#pragma unroll
      for (int sp = 0; sp < SM_MAX_PARTS; ++sp)
        if (sp < n_split) sm_load(p + (size_t)sp * split_stride, part[sp]);
    }
    SmVec<VEC> u;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      if (update) {
        float y = 0.f;
        if (p) {
#pragma unroll
          for (int sp = 0; sp < SM_MAX_PARTS; ++sp)
            if (sp < n_split) y += part[sp].v[e];
        }
        float nx[MAXS];
#pragma unroll
        for (int to = 0; to < MAXS; ++to) {
          if (to >= S) break;
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < MAXS; ++s)
            if (s < S) acc = fmaf(REGW ? r_mix[REGW ? s : 0][REGW ? to : 0] : w_mix[s * S + to], x[s].v[e], acc);
          nx[to] = acc;
        }
        if (p) {          // partials beyond the first few, in order, before the result joins the copies
          for (int sp = SM_MAX_PARTS; sp < n_split; ++sp) y += to_f32(p[(size_t)sp * split_stride + e]);
        }
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
          if (s < S) x[s].v[e] = fmaf(REGW ? r_write[REGW ? s : 0] : w_write[s], y, nx[s]);
      }
      float uu = 0.f;
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) uu = fmaf(REGW ? r_read[REGW ? s : 0] : w_read[s], x[s].v[e], uu);
      u.v[e] = uu;
      ss += uu * uu;
    }
    if (update && write_h) {
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) sm_store(h + (size_t)s * stream_stride + (size_t)t * d + i, x[s]);
    }
    if (out) sm_store(u_buf + i, u);
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float scale = 1.0f / sqrtf(total / (float)d + eps);
  TO* orow = out + (size_t)r * d;
  for (int i = threadIdx.x * VEC; i < d; i += blockDim.x * VEC) {
    SmVec<VEC> u, g;
    sm_load(u_buf + i, u);
    sm_load(gain + i, g);
#pragma unroll
    for (int e = 0; e < VEC; ++e) u.v[e] = (u.v[e] * scale) * g.v[e];
    sm_store(orow + i, u);
  }
}

// h float32 [S, T, d] (copy s at h + s * stream_stride).  delta: null, or n_split partials [T, d] (split_stride
// apart).  mix [S*S] (from, to) and write [S]: the update to apply first, or null for none.  read [S] or null
// (all ones).  rows: null or n_rows row indices into the n_tokens rows of a copy.  out: null or [n_rows, d].
LLMX_API int llmx_stream_mix_norm(float* h, long long stream_stride, int S, const void* delta, int delta_dtype,
                                  int n_split, long long split_stride, const float* mix, const float* write,
                                  const float* read, const int* rows, int n_rows, const float* gain, float eps,
                                  void* out, int out_dtype, int d, int write_h, int n_tokens, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (S <= 0 || S > SM_MAX_STREAMS || d <= 0 || n_split < 1) return LLMX_REFUSED(1);
  if ((mix == nullptr) != (write == nullptr) || (delta && !mix) || (out && !gain)) return LLMX_REFUSED(4);
  const size_t smem = out ? (size_t)d * sizeof(float) : 0;
  if (smem > 200 * 1024) return LLMX_REFUSED(3);
  // four columns per load where every row starts on a 16-byte boundary (8 bytes for bfloat16 rows)
  const bool vec = d % 4 == 0 && stream_stride % 4 == 0 && split_stride % 4 == 0 &&
                   !(((uintptr_t)h | (uintptr_t)delta | (uintptr_t)out | (uintptr_t)gain) & 15);
  // a step of few rows leaves most SMs idle: every row then gets up to 512 threads, so that one pass of loads
  // covers it; a prompt's rows take 256 each and several share an SM
  const int threads = (n_rows <= 64 && d > 1024) ? 512 : 256;
#define GO(TD, TO, VEC, MAXS)                                                                                          \
  do {                                                                                                                 \
    auto kernel = stream_mix_norm_kernel<TD, TO, VEC, MAXS>;                                                           \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
    launch_pdl(kernel, dim3(n_rows), dim3(threads), smem, stream, h, (size_t)stream_stride, S, (const TD*)delta, n_split,  \
               (size_t)split_stride, mix, write, read, rows, gain, eps, (TO*)out, d, write_h, n_tokens);               \
  } while (0)
  // up to four copies: four columns per load where the alignment allows; five to eight: one column (registers)
#define CASE(TD, TO)                          \
  do {                                        \
    if (S > 4) GO(TD, TO, 1, 8);              \
    else if (S > 2) {                         \
      if (vec) GO(TD, TO, 4, 4);              \
      else GO(TD, TO, 1, 4);                  \
    } else if (S == 2) {                      \
      if (vec) GO(TD, TO, 4, 2);              \
      else GO(TD, TO, 1, 2);                  \
    } else {                                  \
      if (vec) GO(TD, TO, 4, 1);              \
      else GO(TD, TO, 1, 1);                  \
    }                                         \
  } while (0)
  if (delta_dtype == LLMX_F32 && out_dtype == LLMX_F32) CASE(float, float);
  else if (delta_dtype == LLMX_F32 && out_dtype == LLMX_BF16) CASE(float, bf16);
  else if (delta_dtype == LLMX_BF16 && out_dtype == LLMX_BF16) CASE(bf16, bf16);
  else if (delta_dtype == LLMX_BF16 && out_dtype == LLMX_F32) CASE(bf16, float);
  else return LLMX_REFUSED(2);
#undef CASE
#undef GO
  return LLMX_LAUNCH_STATUS();
}
