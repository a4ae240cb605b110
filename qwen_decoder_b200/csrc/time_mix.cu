// A recurrent mixer with a matrix state per head and a per-channel, per-token decay, for a flat batch of portions:
//
//   shift_mix  x_s[t] = h[t] + (h[t-1] - h[t]) * mu_s for each of n_mix blends s; h[t-1] of a portion's first token is
//              the request's kept input (its state row), zeros at a sequence's start
//   decay      w[t, c] = exp(-exp(w0[c] + sum_r tanh(a[t, r]) W2[c, r])), a the float32 sums of the low-rank product
//   scan       per (request, head), token by token:  o_t = (S + diag(u) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T
//              S [d, dv] float32 lives in the request's state row, is read once and written once per step
//   finish     out[t, head] = o / sqrt(mean(o^2) + eps) * norm * silu(g) * out_scale, rounded once for the output
//              projection; the last token of every portion leaves its h as the request's kept input
//
// Everything between the projections' float32 sums and ``finish``'s store is float32; the recurrence runs in the
// order of the tokens with a fixed order of additions, so a portion at once and token by token agree bit for bit.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float tm_ld(const void* p, int code, size_t i) {
  return code == QD_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void tm_st(void* p, int code, size_t i, float v) {
  if (code == QD_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------------------------------------------ shift_mix
// grid (ceil(D / 256), T).  h [T, D] (``dtype``); mu float32 [n_mix, D]; out [n_mix, T, D] (``dtype``).
__global__ void __launch_bounds__(256)
tm_shift_mix_kernel(const void* __restrict__ h, int dtype, int T, int D, const float* __restrict__ mu, int n_mix,
                    const float* __restrict__ state, long long state_stride, long long prev_off,
                    const int* __restrict__ token_req, const int* __restrict__ cu_tokens,
                    const int* __restrict__ slots, void* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
  if (c >= D) return;
  const int r = token_req[t];
  const float cur = tm_ld(h, dtype, (size_t)t * D + c);
  const float prev = t > cu_tokens[r] ? tm_ld(h, dtype, (size_t)(t - 1) * D + c)
                                      : state[(size_t)slots[r] * state_stride + prev_off + c];
  const float diff = prev - cur;
  for (int s = 0; s < n_mix; s++)
    tm_st(out, dtype, ((size_t)s * T + t) * D + c, fmaf(diff, mu[(size_t)s * D + c], cur));
}

extern "C" int qd_tm_shift_mix(const void* h, int dtype, int T, int D, const float* mu, int n_mix, const float* state,
                               long long state_stride, long long prev_off, const int* token_req, const int* cu_tokens,
                               const int* slots, void* out, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (T > 65535 || D <= 0 || n_mix <= 0 || !state) return QD_ERR_UNSUPPORTED;     // a step's tokens are far fewer
  qd_launch(tm_shift_mix_kernel, dim3((D + 255) / 256, T), dim3(256), 0, stream, h, dtype, T, D, mu, n_mix, state,
            state_stride, prev_off, token_req, cu_tokens, slots, out);
  return qd_last_error();
}

// ---------------------------------------------------------------------------------------------------------- decay
// grid (ceil(C / 128), ceil(T / TD_TOKENS)), 128 threads.  a float32 [T, lda] (the first R columns); w2t [R, C]
// (``w_dtype``; the transpose of the stored [C, R], so that neighbouring threads read neighbouring numbers);
// w0 float32 [C].  A CTA keeps its 128 channels' columns of w2t in shared memory (float32) for its TD_TOKENS tokens.
#define TD_TOKENS 16

__global__ void __launch_bounds__(128)
tm_decay_kernel(const float* __restrict__ a, long long lda, int T, int R, const void* __restrict__ w2t, int w_dtype,
                const float* __restrict__ w0, int C, float* __restrict__ out) {
  pdl_launch_dependents();
  extern __shared__ float td_sm[];                    // [R][128] weights, then [TD_TOKENS][R] tanh values
  float* ws = td_sm;
  float* th = td_sm + (size_t)R * 128;
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int t0 = blockIdx.y * TD_TOKENS, nt = min(TD_TOKENS, T - t0);
  for (int i = 0; i < R; i++) ws[i * 128 + threadIdx.x] = c < C ? tm_ld(w2t, w_dtype, (size_t)i * C + c) : 0.f;
  const float b = c < C ? w0[c] : 0.f;
  pdl_wait();
  for (int e = threadIdx.x; e < nt * R; e += 128) {
    const int tt = e / R, i = e - tt * R;
    th[e] = tanhf(a[(size_t)(t0 + tt) * lda + i]);
  }
  __syncthreads();
  if (c >= C) return;
  for (int tt = 0; tt < nt; tt++) {
    float z = b;
    for (int i = 0; i < R; i++) z = fmaf(th[tt * R + i], ws[i * 128 + threadIdx.x], z);
    out[(size_t)(t0 + tt) * C + c] = expf(-expf(z));
  }
}

extern "C" int qd_tm_decay(const float* a, long long lda, int T, int R, const void* w2t, int w_dtype, const float* w0,
                           int C, float* out, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = ((size_t)R * 128 + (size_t)TD_TOKENS * R) * sizeof(float);
  if (R <= 0 || C <= 0 || smem > 200 * 1024 || (T + TD_TOKENS - 1) / TD_TOKENS > 65535) return QD_ERR_UNSUPPORTED;
  static size_t raised = 48 * 1024;
  if (smem > raised) {
    cudaFuncSetAttribute(tm_decay_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    raised = smem;
  }
  qd_launch(tm_decay_kernel, dim3((C + 127) / 128, (T + TD_TOKENS - 1) / TD_TOKENS), dim3(128), smem, stream, a, lda, T,
            R, w2t, w_dtype, w0, C, out);
  return qd_last_error();
}

// ----------------------------------------------------------------------------------------------------------- scan
// grid (ceil(dv / 16), H, requests), 256 threads: thread (x = tid & 15, column = tid >> 4) keeps NI elements
// S[x + 16 n, column] of the state in registers.  r, k, w of TM_GROUP tokens arrive in shared memory per group (the
// next group's are fetched into registers while this group is computed, so a group never waits for memory but at the
// start); a token then costs NI x 4 FMAs a thread and a reduction over the 16 threads of a column.
#define TM_GROUP 16

template <int NI>
__global__ void __launch_bounds__(256)
tm_scan_kernel(const float* __restrict__ r_, const float* __restrict__ k_, const float* __restrict__ v_, long long ld,
               const float* __restrict__ w_, const float* __restrict__ u_, int H, int d, int dv,
               float* __restrict__ state, long long state_stride, long long s_off, const int* __restrict__ cu_tokens,
               const int* __restrict__ slots, float* __restrict__ out, int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float tm_sm[];                    // [TM_GROUP][3][16 NI] r, k, w; then [TM_GROUP][16] v
  float* vs = tm_sm + (size_t)TM_GROUP * 3 * 16 * NI;
  const int tid = threadIdx.x, x = tid & 15, jl = tid >> 4;
  const int h = blockIdx.y, req = blockIdx.z, j = blockIdx.x * 16 + jl;
  const bool live = j < dv;
  const int t0 = cu_tokens[req], t1 = cu_tokens[req + 1];
  if (t0 >= t1) return;
  float* S = state + (size_t)slots[req] * state_stride + s_off + (size_t)h * d * dv;
  float s[NI], uu[NI];
#pragma unroll
  for (int n = 0; n < NI; n++) {
    const int i = x + 16 * n;
    s[n] = (live && i < d) ? S[(size_t)i * dv + j] : 0.f;
    uu[n] = i < d ? u_[(size_t)h * d + i] : 0.f;
  }
  // A group's operands in shared memory: [TM_GROUP][3][DP] with DP = 16 NI >= d; places past the portion's end or
  // past d hold r = 0, k = 0, w = 1 (and v = 0), which leave the state and the sums as they are.  Element
  // e = tid + 256 q of it is fetched by this thread, q < PF.
  constexpr int DP = 16 * NI, PF = 3 * NI * TM_GROUP / 16;
  float pf[PF], pv = 0.f;
  auto fetch = [&](int tb) {
    const int nt = min(TM_GROUP, t1 - tb);
#pragma unroll
    for (int q = 0; q < PF; q++) {
      const int e = tid + 256 * q;
      const int tt = e / (3 * DP), rem = e - tt * 3 * DP, which = rem / DP, i = rem - which * DP;
      pf[q] = which == 2 ? 1.f : 0.f;
      if (tt < nt && i < d) {
        const size_t src = (size_t)(tb + tt) * ld + (size_t)h * d + i;
        pf[q] = which == 0 ? r_[src] : which == 1 ? k_[src] : w_[(size_t)(tb + tt) * H * d + (size_t)h * d + i];
      }
    }
    const int tt = tid >> 4, jj = blockIdx.x * 16 + (tid & 15);
    pv = (tt < nt && jj < dv) ? v_[(size_t)(tb + tt) * ld + (size_t)h * dv + jj] : 0.f;
  };
  fetch(t0);
  for (int tb = t0; tb < t1; tb += TM_GROUP) {
    const int nt = min(TM_GROUP, t1 - tb);
    __syncthreads();                                  // the group before is computed
#pragma unroll
    for (int q = 0; q < PF; q++) tm_sm[tid + 256 * q] = pf[q];
    vs[tid] = pv;
    __syncthreads();
    if (tb + TM_GROUP < t1) fetch(tb + TM_GROUP);     // in flight while this group is computed
    float acc[TM_GROUP];
#pragma unroll
    for (int tt = 0; tt < TM_GROUP; tt++) {
      const float vj = vs[tt * 16 + jl];
      const float *rs = tm_sm + tt * 3 * DP, *ks = rs + DP, *ws = ks + DP;
      float a = 0.f;
#pragma unroll
      for (int n = 0; n < NI; n++) {
        const int i = x + 16 * n;
        const float kv = ks[i] * vj;
        a = fmaf(rs[i], fmaf(uu[n], kv, s[n]), a);
        s[n] = fmaf(ws[i], s[n], kv);
      }
      acc[tt] = a;
    }
    // The 16 threads of a column add up their shares of all 16 tokens at once: after the step with distance o a
    // thread keeps the o sums of the half that its bit o of x names, so 15 exchanges do what 64 would, and thread x
    // ends with token x's sum.  A token's sum is the same tree of additions whichever place of a group it has.
#pragma unroll
    for (int o = TM_GROUP / 2; o > 0; o >>= 1) {
      const bool upper = x & o;
#pragma unroll
      for (int i = 0; i < o; i++) {
        const float send = upper ? acc[i] : acc[i + o], keep = upper ? acc[i + o] : acc[i];
        acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
      }
    }
    if (x < nt && live) out[(size_t)(tb + x) * H * dv + (size_t)h * dv + j] = acc[0];
  }
  if (write_state && live) {
#pragma unroll
    for (int n = 0; n < NI; n++) {
      const int i = x + 16 * n;
      if (i < d) S[(size_t)i * dv + j] = s[n];
    }
  }
}

// r, k [T, >= H*d] and v [T, >= H*dv] float32 with rows ``ld`` apart (each pointer at its own first column);
// w float32 [T, H*d] dense; u float32 [H, d]; out float32 [T, H*dv] dense; state float32 rows ``state_stride`` apart,
// the heads' matrices [H, d, dv] at ``s_off``.
extern "C" int qd_tm_scan(const float* r, const float* k, const float* v, long long ld, const float* w, const float* u,
                          int H, int d, int dv, float* state, long long state_stride, long long s_off,
                          const int* cu_tokens, const int* slots, int n_requests, float* out, int write_state,
                          cudaStream_t stream) {
  if (n_requests <= 0) return 0;
  if (H <= 0 || H > 65535 || n_requests > 65535 || d <= 0 || d > 256 || dv <= 0) return QD_ERR_UNSUPPORTED;
  dim3 grid((dv + 15) / 16, H, n_requests);
#define TM_GO(NI)                                                                                                  \
  const size_t smem = ((size_t)TM_GROUP * 3 * 16 * NI + TM_GROUP * 16) * sizeof(float);                            \
  if (smem > 48 * 1024)                                                                                            \
    cudaFuncSetAttribute(tm_scan_kernel<NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
  qd_launch(tm_scan_kernel<NI>, grid, dim3(256), smem, stream, r, k, v, ld, w, u, H, d, dv, state, state_stride,   \
            s_off, cu_tokens, slots, out, write_state)
  if (d <= 16) { TM_GO(1); }
  else if (d <= 32) { TM_GO(2); }
  else if (d <= 64) { TM_GO(4); }
  else if (d <= 128) { TM_GO(8); }
  else { TM_GO(16); }
#undef TM_GO
  return qd_last_error();
}

// --------------------------------------------------------------------------------------------------------- finish
// grid (T, ceil(H / 8)), 256 threads: a warp per head.  o float32 [T, H*dv]; g float32 [T, ldg] gate logits (silu is taken
// here); norm float32 [H*dv]; out rows ``out_stride`` apart in ``out_dtype``.  The last token of a portion copies
// its row of h [T, D] (``h_dtype``) into the request's state row at ``prev_off``.
__global__ void __launch_bounds__(256)
tm_finish_kernel(const float* __restrict__ o, const float* __restrict__ g, long long ldg,
                 const float* __restrict__ norm, int H, int dv, float eps, float out_scale, void* __restrict__ out,
                 int out_dtype, long long out_stride, const void* __restrict__ h, int h_dtype, int D,
                 float* __restrict__ state, long long state_stride, long long prev_off,
                 const int* __restrict__ token_req, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                 int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hd = blockIdx.y * 8 + warp;
  if (hd < H) {
    const size_t base = (size_t)t * H * dv + (size_t)hd * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) { const float y = o[base + i]; ss = fmaf(y, y, ss); }
    const float f = out_scale / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
      const float z = g[(size_t)t * ldg + (size_t)hd * dv + i];
      const float gate = z / (1.0f + expf(-z));
      tm_st(out, out_dtype, (size_t)t * out_stride + (size_t)hd * dv + i, o[base + i] * f * norm[hd * dv + i] * gate);
    }
  }
  if (!write_state || blockIdx.y != 0) return;
  const int r = token_req[t];
  if (t != cu_tokens[r + 1] - 1) return;
  float* prev = state + (size_t)slots[r] * state_stride + prev_off;
  for (int c = threadIdx.x; c < D; c += blockDim.x) prev[c] = tm_ld(h, h_dtype, (size_t)t * D + c);
}

extern "C" int qd_tm_finish(const float* o, const float* g, long long ldg, const float* norm, int T, int H, int dv,
                            float eps, float out_scale, void* out, int out_dtype, long long out_stride, const void* h,
                            int h_dtype, int D, float* state, long long state_stride, long long prev_off,
                            const int* token_req, const int* cu_tokens, const int* slots, int write_state,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dv <= 0 || !state) return QD_ERR_UNSUPPORTED;
  if ((H + 7) / 8 > 65535) return QD_ERR_UNSUPPORTED;
  qd_launch(tm_finish_kernel, dim3(T, (H + 7) / 8), dim3(256), 0, stream, o, g, ldg, norm, H, dv, eps, out_scale, out, out_dtype,
            out_stride, h, h_dtype, D, state, state_stride, prev_off, token_req, cu_tokens, slots, write_state);
  return qd_last_error();
}
