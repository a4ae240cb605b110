// Kernels of a pre-norm layer whose branches join through a gate, whose mixer reads its input through a short
// causal convolution, and of a loop of layers that takes the embedding output in again:
//
//   gated_add_norm   x[s] += sigmoid(g[s] + b) * delta[s] (element by element; g float32 logits, b a bias per channel
//                    or none; delta in the engine's
//                    dtype or float32 partial sums that are added up here), then optionally out[r] = x[s] /
//                    sqrt(mean(x[s]^2) + eps) * w  with s = rows[r] (or r)                          float32 arithmetic
//   short_conv       y[t, c] = (residual ? u[t, c] : 0) + sum_j w[c, j] * u[t - taps + 1 + j, c] per request; inputs
//                    before the portion's first token come from the request's state row (the last taps - 1 inputs,
//                    oldest first, float32), zeros at a sequence's start (a fresh state row is zero)
//   short_conv_state moves every request's state row on by its portion, whatever the portion's length (a step of single
//                    tokens, one per request, needs no such launch: the convolution's own thread moves its channel on)
//   concat_round     out[t] = [a[t] | b[t]] in the engine's dtype, from two float32 rows
//   plain_act        out = act(z) element by element (the tanh form of gelu), from float32 sums
#include "common.cuh"
#include "short_conv.cuh"

// ---------------------------------------------------------------------------------------------- gated add + norm
template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
gated_add_norm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_parts, size_t part_stride,
                      const float* __restrict__ gate, const float* __restrict__ gate_bias,
                      const float* __restrict__ w, TO* __restrict__ out,
                      const int* __restrict__ rows, int D, float eps, int write_back) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];          // D values + 40 scratch
  float* v = sm;
  float* scratch = sm + D;
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float* xr = x + s * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float a = xr[i];
    if (delta) {
      float dsum = to_float(delta[s * D + i]);
      for (int p = 1; p < n_parts; p++) dsum += to_float(delta[p * part_stride + s * D + i]);
      if (gate) dsum *= 1.0f / (1.0f + expf(-(gate[s * D + i] + (gate_bias ? gate_bias[i] : 0.f))));
      a += dsum;
      if (write_back) xr[i] = a;
    }
    v[i] = a;
    ss = fmaf(a, a, ss);
  }
  if (!w) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  TO* o = out + (size_t)r * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = from_float<TO>(v[i] * inv * w[i]);
}

// The same with four elements a thread and turn, a row's operands in registers (D a multiple of 4, at most 8192).
template <typename TD, typename TO, int VPT>
__global__ void __launch_bounds__(1024)
gated_add_norm_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_parts, size_t part_stride,
                          const float* __restrict__ gate, const float* __restrict__ gate_bias,
                          const float* __restrict__ w, TO* __restrict__ out,
                          const int* __restrict__ rows, int D, float eps, int write_back) {
  pdl_launch_dependents();
  const int n4 = D >> 2;
  float4 v[VPT], wv[VPT];
#pragma unroll
  for (int q = 0; q < VPT; q++) {
    const int i4 = threadIdx.x + q * blockDim.x;
    wv[q] = (w && i4 < n4) ? reinterpret_cast<const float4*>(w)[i4] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  __shared__ float scratch[40];
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float ss = 0.f;
#pragma unroll
  for (int q = 0; q < VPT; q++) {
    const int i4 = threadIdx.x + q * blockDim.x;
    v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i4 < n4) {
      float4 a = reinterpret_cast<const float4*>(x + s * D)[i4];
      if (delta) {
        float4 d;
        if (sizeof(TD) == 4) {
          const float* dp = reinterpret_cast<const float*>(delta) + s * D;
          d = reinterpret_cast<const float4*>(dp)[i4];
          for (int p = 1; p < n_parts; p++) {
            const float4 e = reinterpret_cast<const float4*>(dp + (size_t)p * part_stride)[i4];
            d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
          }
        } else {
          const bf16* dp = reinterpret_cast<const bf16*>(delta) + s * D + 4 * (size_t)i4;
          const uint2 raw = *reinterpret_cast<const uint2*>(dp);
          const __nv_bfloat162 d0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 d1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          d = make_float4(__low2float(d0), __high2float(d0), __low2float(d1), __high2float(d1));
        }
        if (gate) {
          float4 g = reinterpret_cast<const float4*>(gate + s * D)[i4];
          if (gate_bias) {
            const float4 b = reinterpret_cast<const float4*>(gate_bias)[i4];
            g.x += b.x; g.y += b.y; g.z += b.z; g.w += b.w;
          }
          d.x *= 1.0f / (1.0f + expf(-g.x)); d.y *= 1.0f / (1.0f + expf(-g.y));
          d.z *= 1.0f / (1.0f + expf(-g.z)); d.w *= 1.0f / (1.0f + expf(-g.w));
        }
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        if (write_back) reinterpret_cast<float4*>(x + s * D)[i4] = a;
      }
      v[q] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  if (!w) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
  for (int q = 0; q < VPT; q++) {
    const int i4 = threadIdx.x + q * blockDim.x;
    if (i4 < n4) {
      const float4 ww = wv[q];
      const float o0 = v[q].x * inv * ww.x, o1 = v[q].y * inv * ww.y, o2 = v[q].z * inv * ww.z, o3 = v[q].w * inv * ww.w;
      if (sizeof(TO) == 4) {
        reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)r * D)[i4] = make_float4(o0, o1, o2, o3);
      } else {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&p0);
        raw.y = *reinterpret_cast<unsigned*>(&p1);
        *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + (size_t)r * D + 4 * (size_t)i4) = raw;
      }
    }
  }
}

// x float32 [T, D]; delta [T, D] (``delta_dtype``) or float32 [n_parts, T, D], or null; gate float32 [T, D] or null, with
// gate_bias float32 [D] (or null) added to every row of it; w float32 [D] or null (no norm: out is not written); rows
// int32 [n_rows] or null.
extern "C" int qd_gated_add_norm(float* x, const void* delta, int delta_dtype, int n_parts, long long part_stride,
                                 const float* gate, const float* gate_bias, const float* w, void* out, int out_dtype,
                                 const int* rows,
                                 int n_rows, int D, float eps, int write_back, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (delta && delta_dtype != QD_F32 && (delta_dtype != QD_BF16 || n_parts != 1)) return QD_ERR_UNSUPPORTED;
  if (w && out_dtype != QD_F32 && out_dtype != QD_BF16) return QD_ERR_UNSUPPORTED;
  const bool df = !delta || delta_dtype == QD_F32, of = !w || out_dtype == QD_F32;
  const bool al = !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)gate | (uintptr_t)gate_bias | (uintptr_t)w |
                    (uintptr_t)out) & 15);
  if (D % 4 == 0 && D <= 8192 && al) {
    const int n4 = D / 4;
    int threads = n4 <= 1024 ? ((n4 + 31) / 32) * 32 : 1024;
#define GA_VEC(TD, TO)                                                                                          \
  do {                                                                                                          \
    if (n4 <= 1024)                                                                                             \
      qd_launch(gated_add_norm_vec_kernel<TD, TO, 1>, dim3(n_rows), dim3(threads), 0, stream, x, (const TD*)delta, \
                n_parts, (size_t)part_stride, gate, gate_bias, w, (TO*)out, rows, D, eps, write_back);                     \
    else                                                                                                        \
      qd_launch(gated_add_norm_vec_kernel<TD, TO, 2>, dim3(n_rows), dim3(threads), 0, stream, x, (const TD*)delta, \
                n_parts, (size_t)part_stride, gate, gate_bias, w, (TO*)out, rows, D, eps, write_back);                     \
  } while (0)
    if (df && of) GA_VEC(float, float);
    else if (df) GA_VEC(float, bf16);
    else if (of) GA_VEC(bf16, float);
    else GA_VEC(bf16, bf16);
#undef GA_VEC
    return qd_last_error();
  }
  const size_t smem = (size_t)(D + 40) * sizeof(float);
  if (smem > 200 * 1024) return QD_ERR_UNSUPPORTED;
#define GA_GO(TD, TO)                                                                                          \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(gated_add_norm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    qd_launch(gated_add_norm_kernel<TD, TO>, dim3(n_rows), dim3(256), smem, stream, x, (const TD*)delta, n_parts, \
              (size_t)part_stride, gate, gate_bias, w, (TO*)out, rows, D, eps, write_back);                               \
  } while (0)
  if (df && of) GA_GO(float, float);
  else if (df) GA_GO(float, bf16);
  else if (of) GA_GO(bf16, float);
  else GA_GO(bf16, bf16);
#undef GA_GO
  return qd_last_error();
}

// ---------------------------------------------------------------------------------------------- short convolution
// grid (ceil(C / 256), T): one thread per (token, channel).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
short_conv_kernel(const TI* __restrict__ u, long long ldu, int C, int taps, const float* __restrict__ w,
                  float* state, long long state_stride, long long state_off,
                  const int* __restrict__ token_req, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                  TO* __restrict__ out, long long ldo, int residual, int advance) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
  if (c >= C) return;
  const int r = token_req[t];
  float* st = state ? state + (size_t)slots[r] * state_stride + state_off : nullptr;
  float y = short_conv_at(u, ldu, C, taps, w, st, cu_tokens[r], t, c);
  if (residual) y += to_float(u[(size_t)t * ldu + c]);
  out[(size_t)t * ldo + c] = from_float<TO>(y);
  // every request brings one token: this thread alone reads and writes channel c of its request's kept inputs
  if (advance) short_conv_advance(u, ldu, C, taps, st, t, t + 1, c);
}

// grid (ceil(C / 256), requests): one thread per (request, channel) moves the channel's taps - 1 kept inputs on.
template <typename TI>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const TI* __restrict__ u, long long ldu, int C, int taps, float* __restrict__ state,
                        long long state_stride, long long state_off, const int* __restrict__ cu_tokens,
                        const int* __restrict__ slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
  if (c >= C) return;
  short_conv_advance(u, ldu, C, taps, state + (size_t)slots[r] * state_stride + state_off, cu_tokens[r],
                     cu_tokens[r + 1], c);
}

// u [T, >= C] rows ldu apart (``in_dtype``); w float32 [C, taps]; state float32 rows ``state_stride`` apart, this
// convolution's (taps - 1) x C kept inputs at ``state_off`` (null with taps == 1); out rows ldo apart.
extern "C" int qd_short_conv(const void* u, int in_dtype, long long ldu, int C, int taps, const float* w,
                             float* state, long long state_stride, long long state_off, const int* token_req,
                             const int* cu_tokens, const int* slots, void* out, int out_dtype, long long ldo, int T,
                             int n_requests, int residual, int update_state, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || C <= 0 || T > 65535 * 64 || (taps > 1 && !state)) return QD_ERR_UNSUPPORTED;
  dim3 grid((C + 255) / 256, T);
  if (grid.y > 65535) return QD_ERR_UNSUPPORTED;
  // single tokens (one per request): the convolution's own launch moves the kept inputs on
  const int advance = update_state && taps > 1 && T == n_requests;
#define SC_GO(TI, TO)                                                                                          \
  qd_launch(short_conv_kernel<TI, TO>, grid, dim3(256), 0, stream, (const TI*)u, ldu, C, taps, w, state,       \
            state_stride, state_off, token_req, cu_tokens, slots, (TO*)out, ldo, residual, advance)
  if (in_dtype == QD_F32 && out_dtype == QD_F32) SC_GO(float, float);
  else if (in_dtype == QD_F32 && out_dtype == QD_BF16) SC_GO(float, bf16);
  else if (in_dtype == QD_BF16 && out_dtype == QD_BF16) SC_GO(bf16, bf16);
  else if (in_dtype == QD_BF16 && out_dtype == QD_F32) SC_GO(bf16, float);
  else return QD_ERR_UNSUPPORTED;
#undef SC_GO
  if (update_state && taps > 1 && !advance) {
    dim3 g2((C + 255) / 256, n_requests);
    if (in_dtype == QD_F32)
      qd_launch(short_conv_state_kernel<float>, g2, dim3(256), 0, stream, (const float*)u, ldu, C, taps, state,
                state_stride, state_off, cu_tokens, slots);
    else
      qd_launch(short_conv_state_kernel<bf16>, g2, dim3(256), 0, stream, (const bf16*)u, ldu, C, taps, state,
                state_stride, state_off, cu_tokens, slots);
  }
  return qd_last_error();
}

// The state update alone (for a caller whose own kernel made the convolution).
extern "C" int qd_short_conv_state(const void* u, int in_dtype, long long ldu, int C, int taps, float* state,
                                   long long state_stride, long long state_off, const int* cu_tokens,
                                   const int* slots, int n_requests, cudaStream_t stream) {
  if (n_requests <= 0 || taps <= 1) return 0;
  if (n_requests > 65535 || !state) return QD_ERR_UNSUPPORTED;
  dim3 g2((C + 255) / 256, n_requests);
  if (in_dtype == QD_F32)
    qd_launch(short_conv_state_kernel<float>, g2, dim3(256), 0, stream, (const float*)u, ldu, C, taps, state,
              state_stride, state_off, cu_tokens, slots);
  else if (in_dtype == QD_BF16)
    qd_launch(short_conv_state_kernel<bf16>, g2, dim3(256), 0, stream, (const bf16*)u, ldu, C, taps, state,
              state_stride, state_off, cu_tokens, slots);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// ---------------------------------------------------------------------------------------------- concat, activation
template <typename TO>
__global__ void __launch_bounds__(256)
concat_round_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out, int D, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;     // over [T, 2 D]
  if (i >= n) return;
  const size_t t = i / (2 * (size_t)D);
  const int c = (int)(i - t * 2 * (size_t)D);
  out[i] = from_float<TO>(c < D ? a[t * D + c] : b[t * D + (c - D)]);
}

extern "C" int qd_concat_round(const float* a, const float* b, void* out, int out_dtype, int T, int D,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t n = (size_t)T * 2 * D;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (out_dtype == QD_F32) qd_launch(concat_round_kernel<float>, dim3(blocks), dim3(256), 0, stream, a, b, (float*)out, D, n);
  else if (out_dtype == QD_BF16) qd_launch(concat_round_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, a, b, (bf16*)out, D, n);
  else return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// out[t, :] = act(sum of the n_parts float32 partial sums z[p, t, :]); act 0: the tanh form of gelu.
template <typename TO>
__global__ void __launch_bounds__(256)
plain_act_kernel(const float* __restrict__ z, int n_parts, size_t part_stride, TO* __restrict__ out, size_t n, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = z[i];
  for (int p = 1; p < n_parts; p++) v += z[p * part_stride + i];
  out[i] = from_float<TO>(gelu_tanh(v));
}

extern "C" int qd_plain_act(const float* z, int n_parts, long long part_stride, void* out, int out_dtype, long long n,
                            int act, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (act != 0) return QD_ERR_UNSUPPORTED;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (out_dtype == QD_F32)
    qd_launch(plain_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, z, n_parts, (size_t)part_stride, (float*)out, (size_t)n, act);
  else if (out_dtype == QD_BF16)
    qd_launch(plain_act_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, z, n_parts, (size_t)part_stride, (bf16*)out, (size_t)n, act);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
