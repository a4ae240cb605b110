// Differential grouped-query attention: every head runs TWO softmax maps over the same values and keeps their
// difference.
//
//   prep     the stacked projection [q (H * 2d) | k (G * 2d) | v (G * vd) | ...] (float32) passes a short causal
//            convolution per channel (``short_conv.cuh``; the request's kept inputs come from its state row); q goes
//            to a dense [T, H * 2d] tensor, k and v to the token's slot of the paged cache.  A head's query and a
//            kv head's key are laid out [map 1 (d) | map 2 (d)]: a cached key is one row of 2d numbers.
//   attend   s_m,j = (q_m . k_m,j) * scale, then cap * tanh(s / cap) when a cap is given; p_m = softmax over the keys
//            j <= position (or the last ``window``); a_m = sum_j p_m,j v_j   (m = 1, 2; both maps read the same v)
//            o = a_1 - lambda * a_2;  o <- o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate[t, h])
//            lambda, out_scale: one number each for the layer.  Scores, weights and the norm are float32.
//
// A page of the cache holds the keys [G, page_size, 2d] and then the values [G, page_size, vd].
// The generic kernel (one warp per (token, head), float32 FMA, any sizes, tiles of 32 keys counted from key 0) serves
// float32 and odd sizes; the tensor-core kernel below it serves bfloat16.
#include "common.cuh"
#include "short_conv.cuh"
#include <math.h>

#define AD_MAX_VD 512
#define AD_WARPS 4

// ------------------------------------------------------------------------------------------------------------- prep
// One thread per (token, channel) of the first ``C`` = Cq + Ck + Cv columns of u.
template <typename TC>
__global__ void __launch_bounds__(256)
diff_conv_write_kernel(const float* __restrict__ u, long long ldu, int Cq, int Ck, int Cv, int taps,
                       const float* __restrict__ w, const float* __restrict__ state, long long state_stride,
                       long long state_off, const int* __restrict__ token_req, const int* __restrict__ cu_tokens,
                       const int* __restrict__ slots, TC* __restrict__ q_out, TC* __restrict__ kv,
                       const int* __restrict__ slot_map, int page_size, int G, int d2, int vd, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int C = Cq + Ck + Cv;
  const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
  if (c >= C) return;
  if (c >= Cq && !write_kv) return;
  float y;
  if (taps > 0) {
    const int r = token_req[t];
    const float* st = state ? state + (size_t)slots[r] * state_stride + state_off : nullptr;
    y = short_conv_at(u, ldu, C, taps, w, st, cu_tokens[r], t, c);
  } else {
    y = u[(size_t)t * ldu + c];
  }
  if (c < Cq) {
    q_out[(size_t)t * Cq + c] = from_float<TC>(y);
    return;
  }
  const size_t slot = (size_t)slot_map[t], page = slot / page_size, off = slot - page * page_size;
  const size_t page_elems = (size_t)G * page_size * (d2 + vd);
  if (c < Cq + Ck) {
    const int k = c - Cq, g = k / d2, i = k - g * d2;
    kv[page * page_elems + ((size_t)g * page_size + off) * d2 + i] = from_float<TC>(y);
  } else {
    const int k = c - Cq - Ck, g = k / vd, i = k - g * vd;
    kv[page * page_elems + (size_t)G * page_size * d2 + ((size_t)g * page_size + off) * vd + i] = from_float<TC>(y);
  }
}

__global__ void __launch_bounds__(256)
diff_conv_state_kernel(const float* __restrict__ u, long long ldu, int C, int taps, float* __restrict__ state,
                       long long state_stride, long long state_off, const int* __restrict__ cu_tokens,
                       const int* __restrict__ slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
  if (c >= C) return;
  short_conv_advance(u, ldu, C, taps, state + (size_t)slots[r] * state_stride + state_off, cu_tokens[r],
                     cu_tokens[r + 1], c);
}

// u float32 [T, >= Cq + Ck + Cv] rows ldu apart; w float32 [Cq + Ck + Cv, taps] (taps 0: no convolution); state
// float32 rows state_stride apart with this convolution's (taps - 1) x C kept inputs at state_off; q_out [T, Cq] and
// kv in ``dtype``.  With ``write`` the keys and values are written and the state is moved on by the portion.
extern "C" int qd_diff_conv_write(const float* u, long long ldu, int H, int G, int d, int vd, int taps, const float* w,
                                  float* state, long long state_stride, long long state_off, const int* token_req,
                                  const int* cu_tokens, const int* slots, void* q_out, void* kv, int dtype,
                                  const int* slot_map, int page_size, int T, int n_requests, int write,
                                  cudaStream_t stream) {
  if (T <= 0) return 0;
  const int d2 = 2 * d, Cq = H * d2, Ck = G * d2, Cv = G * vd, C = Cq + Ck + Cv;
  if (taps < 0 || (taps > 1 && !state) || T > 65535 || n_requests > 65535 || page_size <= 0) return QD_ERR_UNSUPPORTED;
  dim3 grid((C + 255) / 256, T);
  if (dtype == QD_F32)
    qd_launch(diff_conv_write_kernel<float>, grid, dim3(256), 0, stream, u, ldu, Cq, Ck, Cv, taps, w,
              (const float*)state, state_stride, state_off, token_req, cu_tokens, slots, (float*)q_out, (float*)kv,
              slot_map, page_size, G, d2, vd, write);
  else if (dtype == QD_BF16)
    qd_launch(diff_conv_write_kernel<bf16>, grid, dim3(256), 0, stream, u, ldu, Cq, Ck, Cv, taps, w,
              (const float*)state, state_stride, state_off, token_req, cu_tokens, slots, (bf16*)q_out, (bf16*)kv,
              slot_map, page_size, G, d2, vd, write);
  else
    return QD_ERR_UNSUPPORTED;
  if (write && taps > 1)
    qd_launch(diff_conv_state_kernel, dim3((C + 255) / 256, n_requests), dim3(256), 0, stream, u, ldu, C, taps, state,
              state_stride, state_off, cu_tokens, slots);
  return qd_last_error();
}

// ----------------------------------------------------------------------------------------------------------- attend
struct DiffParams {
  float scale, cap, lambda, eps, out_scale;   // cap 0: scores are not capped
};

__device__ __forceinline__ float ad_cap(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

// The last step of a head, shared by the kernels: from the two maps' sums (already divided by their softmax sums) in
// ``o`` (lane i holds elements i, i + 32, ...), the difference, its unit norm, the constant and the head's gate.
template <typename T>
__device__ __forceinline__ void ad_finish(float* a1, const float* a2, int vd, int lane, const DiffParams& P,
                                          float gate_logit, T* orow) {
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < AD_MAX_VD / 32; i++) {
    const int idx = lane + 32 * i;
    a1[i] = idx < vd ? a1[i] - P.lambda * a2[i] : 0.f;
    ss = fmaf(a1[i], a1[i], ss);
  }
  ss = warp_sum(ss);
  const float f = P.out_scale / sqrtf(ss / (float)vd + P.eps) / (1.0f + expf(-gate_logit));
#pragma unroll
  for (int i = 0; i < AD_MAX_VD / 32; i++) {
    const int idx = lane + 32 * i;
    if (idx < vd) orow[idx] = from_float<T>(a1[i] * f);
  }
}

template <typename T>
__global__ void __launch_bounds__(AD_WARPS * 32)
diff_attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ kv,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_req,
                              const int* __restrict__ positions, int n_tokens, int H, int G, int d, int vd,
                              int page_size, int window, DiffParams P, const float* __restrict__ gate, long long ldg) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AD_WARPS + warp;
  if (item >= (long long)n_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const int g = h / (H / G), d2 = 2 * d;
  float* qs = smem + (size_t)warp * d2;
  const T* qr = q + ((size_t)t * H + h) * d2;
  for (int i = lane; i < d2; i += 32) qs[i] = to_float(qr[i]);
  __syncwarp();

  const int pos = positions[t];
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  const int key_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const size_t page_elems = (size_t)G * page_size * (d2 + vd);
  const size_t k_head = (size_t)g * page_size * d2;
  const size_t v_head = (size_t)G * page_size * d2 + (size_t)g * page_size * vd;

  float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f;
  float o1[AD_MAX_VD / 32], o2[AD_MAX_VD / 32];
#pragma unroll
  for (int i = 0; i < AD_MAX_VD / 32; i++) o1[i] = o2[i] = 0.f;

  for (int base = key_lo & ~31; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key >= key_lo && key <= pos;
    float s1 = -INFINITY, s2 = -INFINITY;
    if (valid) {
      const int page = bt[key / page_size];
      const T* kr = kv + (size_t)page * page_elems + k_head + (size_t)(key % page_size) * d2;
      float a = 0.f, b = 0.f;
      for (int i = 0; i < d; i++) {
        a = fmaf(qs[i], to_float(kr[i]), a);
        b = fmaf(qs[d + i], to_float(kr[d + i]), b);
      }
      s1 = ad_cap(a * P.scale, P.cap);
      s2 = ad_cap(b * P.scale, P.cap);
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);          // -inf on the first tile gives 0
    const float p1 = valid ? expf(s1 - n1) : 0.f, p2 = valid ? expf(s2 - n2) : 0.f;
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
    m1 = n1; m2 = n2;
#pragma unroll
    for (int i = 0; i < AD_MAX_VD / 32; i++) { o1[i] *= c1; o2[i] *= c2; }
    const int jend = pos - base + 1 < 32 ? pos - base + 1 : 32;
    for (int j = 0; j < jend; j++) {
      const float w1 = __shfl_sync(0xffffffffu, p1, j), w2 = __shfl_sync(0xffffffffu, p2, j);
      const int kj = base + j;
      if (kj < key_lo) continue;
      const int page = bt[kj / page_size];
      const T* vr = kv + (size_t)page * page_elems + v_head + (size_t)(kj % page_size) * vd;
#pragma unroll
      for (int i = 0; i < AD_MAX_VD / 32; i++) {
        const int idx = lane + 32 * i;
        if (idx < vd) {
          const float v = to_float(vr[idx]);
          o1[i] = fmaf(w1, v, o1[i]);
          o2[i] = fmaf(w2, v, o2[i]);
        }
      }
    }
  }
  const float i1 = 1.0f / l1, i2 = 1.0f / l2;
#pragma unroll
  for (int i = 0; i < AD_MAX_VD / 32; i++) { o1[i] *= i1; o2[i] *= i2; }
  ad_finish<T>(o1, o2, vd, lane, P, gate ? gate[(size_t)t * ldg + h] : INFINITY, out + ((size_t)t * H + h) * vd);
}

// q [n_tokens, H * 2d] and out [n_tokens, H * vd] dense in ``dtype``; kv pages of [G, page_size, 2d] keys then
// [G, page_size, vd] values; gate float32 logits, element (t, h) at gate[t * ldg + h], or null (no gate).
extern "C" int qd_diff_attention_generic(const void* q, void* out, const void* kv, int dtype, const int* block_table,
                                         int max_blocks, const int* token_req, const int* positions, int n_tokens,
                                         int H, int G, int d, int vd, int page_size, float scale, float cap,
                                         float lambda, float eps, float out_scale, int window, const float* gate,
                                         long long ldg, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || vd <= 0 || vd > AD_MAX_VD || G <= 0 || H % G != 0 || page_size <= 0 || 2 * d > 2048)
    return QD_ERR_UNSUPPORTED;
  const DiffParams P = {scale, cap, lambda, eps, out_scale};
  const long long items = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + AD_WARPS - 1) / AD_WARPS);
  const size_t smem = (size_t)AD_WARPS * 2 * d * sizeof(float);
  if (dtype == QD_F32)
    qd_launch(diff_attention_generic_kernel<float>, dim3(blocks), dim3(AD_WARPS * 32), smem, stream, (const float*)q,
              (float*)out, (const float*)kv, block_table, max_blocks, token_req, positions, n_tokens, H, G, d, vd,
              page_size, window, P, gate, ldg);
  else if (dtype == QD_BF16)
    qd_launch(diff_attention_generic_kernel<bf16>, dim3(blocks), dim3(AD_WARPS * 32), smem, stream, (const bf16*)q,
              (bf16*)out, (const bf16*)kv, block_table, max_blocks, token_req, positions, n_tokens, H, G, d, vd,
              page_size, window, P, gate, ldg);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
