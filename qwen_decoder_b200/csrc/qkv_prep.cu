// What stands between the stacked q/k/v product and attention, for a flat batch of portions, one CTA per token:
//
//   u [T, ld] float32 sums, a row = [q (H*d) | k (G*d) | v (G*vd) | ...]   (a bias was added by the product)
//   conv      with ``taps`` > 0 every channel of q, k and v passes a short causal convolution over time
//             (``short_conv.cuh``: inputs before the portion come from the request's kept inputs in its state row)
//   whole     ``norm_mode`` 1: q <- q / sqrt(mean(q^2) + eps) * wq over the WHOLE projection (all heads at once;
//             wq [H*d]), k alike with wk [G*d]; before the rotation
//   turn      the first ``rotary_dim`` elements of every head of q and k turn by the token's position (table rows
//             of cos and sin; pairs (2i, 2i+1) with ``pairing`` 0, (i, i + rotary_dim/2) with 1)
//   head      ``norm_mode`` 2: every head of q and k is divided by sqrt(mean(head^2) + eps), no weight;
//             ``norm_after`` says whether that happens after the rotation or before it
//   write     q to a dense [T, H*d] tensor, k and v to the token's slot of the paged cache
//             (a page: keys [G, page_size, d], then values [G, page_size, vd])
//
// Everything is float32 until the stores.  The order of every sum depends on the sizes only.
#include "common.cuh"
#include "short_conv.cuh"
#include <math.h>

#define QP_MAX_D 512
#define QP_THREADS 256

__device__ __forceinline__ void qp_st(void* p, int code, size_t i, float v) {
  if (code == QD_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
}

// The two elements of pair j of a head: (2j, 2j+1), or with half-split pairing (j, j + half) inside the rotated part
// (pairs past it cover the elements from 2 half on, two by two).
__device__ __forceinline__ void qp_pair(int pairing, int half, int j, int& ia, int& ib) {
  if (pairing == 1 && j < half) { ia = j; ib = j + half; }
  else { ia = 2 * j; ib = 2 * j + 1; }
}

struct QkvPrep {
  const float* u; long long ld;
  int H, G, d, vd;
  int taps; const float* conv_w; float* state; long long state_stride, state_off;
  const int *token_req, *cu_tokens, *slots; int advance;
  int norm_mode, norm_after; const float *wq, *wk; float eps;
  int rotary_dim, pairing; const float *cos_t, *sin_t; const int* positions;
  void* q_out; int q_dtype; void* kv; int kv_dtype; const int* slot_map; int page_size, write_kv;
};

// NP: pairs of a head that a lane holds (d <= 64 NP); the CTA's threads (a multiple of 32) share a token's channels.
template <int NP>
__global__ void __launch_bounds__(1024)
qkv_prep_kernel(QkvPrep a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float qp_sm[];                    // C values, then 33 of scratch
  const int H = a.H, G = a.G, d = a.d, vd = a.vd;
  const int nq = H * d, nk = G * d, C = nq + nk + G * vd;
  float* row = qp_sm;
  float* scratch = qp_sm + C;
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = a.token_req[t];
  float* kept = (a.taps > 1) ? a.state + (size_t)a.slots[r] * a.state_stride + a.state_off : nullptr;
  const int first = a.cu_tokens[r];
  float ssq = 0.f, ssk = 0.f;
  for (int c = tid; c < C; c += blockDim.x) {
    const float y = a.taps > 0 ? short_conv_at(a.u, a.ld, C, a.taps, a.conv_w, kept, first, t, c)
                               : a.u[(size_t)t * a.ld + c];
    row[c] = y;
    if (c < nq) ssq = fmaf(y, y, ssq);
    else if (c < nq + nk) ssk = fmaf(y, y, ssk);
  }
  float fq = 1.f, fk = 1.f;
  if (a.norm_mode == 1) {
    fq = 1.0f / sqrtf(block_sum(ssq, scratch) / (float)nq + a.eps);
    fk = 1.0f / sqrtf(block_sum(ssk, scratch) / (float)nk + a.eps);
  }
  __syncthreads();
  // every request brings one token: channel c's kept inputs were read by this thread alone, which now moves them on
  if (a.advance)
    for (int c = tid; c < C; c += blockDim.x) short_conv_advance(a.u, a.ld, C, a.taps, kept, t, t + 1, c);

  size_t page = 0, off = 0;
  if (a.write_kv) {
    const size_t slot = (size_t)a.slot_map[t];
    page = slot / a.page_size;
    off = slot - page * a.page_size;
  }
  const size_t page_elems = (size_t)G * a.page_size * (d + vd);
  const int pos = a.positions[t];
  const int half = a.rotary_dim / 2, pairs = d / 2;
  for (int s = warp; s < H + G; s += blockDim.x >> 5) {
    const bool is_q = s < H;
    if (!is_q && !a.write_kv) continue;
    const int base = is_q ? s * d : nq + (s - H) * d;           // the head's first channel in the row
    const float* w = a.norm_mode == 1 ? (is_q ? a.wq + s * d : a.wk + (s - H) * d) : nullptr;
    const float f = is_q ? fq : fk;
    float x[NP], y[NP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NP; i++) {
      const int j = lane + 32 * i;
      x[i] = y[i] = 0.f;
      if (j >= pairs) continue;
      int ia, ib;
      qp_pair(a.pairing, half, j, ia, ib);
      float xa = row[base + ia], yb = row[base + ib];
      if (w) { xa *= f * w[ia]; yb *= f * w[ib]; }
      if (a.norm_mode == 2 && !a.norm_after) ss = fmaf(xa, xa, fmaf(yb, yb, ss));
      x[i] = xa; y[i] = yb;
    }
    if (a.norm_mode == 2 && !a.norm_after) {
      const float fh = 1.0f / sqrtf(warp_sum(ss) / (float)d + a.eps);
#pragma unroll
      for (int i = 0; i < NP; i++) { x[i] *= fh; y[i] *= fh; }
    }
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < NP; i++) {
      const int j = lane + 32 * i;
      if (j < half) {
        const float c = a.cos_t[(size_t)pos * half + j], sn = a.sin_t[(size_t)pos * half + j];
        const float xr = x[i] * c - y[i] * sn, yr = y[i] * c + x[i] * sn;
        x[i] = xr; y[i] = yr;
      }
      ss = fmaf(x[i], x[i], fmaf(y[i], y[i], ss));
    }
    float fh = 1.f;
    if (a.norm_mode == 2 && a.norm_after) fh = 1.0f / sqrtf(warp_sum(ss) / (float)d + a.eps);
    const size_t dst = is_q ? (size_t)t * nq + (size_t)s * d
                            : page * page_elems + ((size_t)(s - H) * a.page_size + off) * d;
    void* out = is_q ? a.q_out : a.kv;
    const int oc = is_q ? a.q_dtype : a.kv_dtype;
#pragma unroll
    for (int i = 0; i < NP; i++) {
      const int j = lane + 32 * i;
      if (j >= pairs) continue;
      int ia, ib;
      qp_pair(a.pairing, half, j, ia, ib);
      qp_st(out, oc, dst + ia, x[i] * fh);
      qp_st(out, oc, dst + ib, y[i] * fh);
    }
  }
  if (!a.write_kv) return;
  const size_t vdst = page * page_elems + (size_t)G * a.page_size * d;
  for (int c = tid; c < G * vd; c += blockDim.x) {
    const int g = c / vd, i = c - g * vd;
    qp_st(a.kv, a.kv_dtype, vdst + ((size_t)g * a.page_size + off) * vd + i, row[nq + nk + c]);
  }
}

// grid (ceil(C / 256), requests): one thread per (request, channel) moves the channel's taps - 1 kept inputs on.
__global__ void __launch_bounds__(256)
qkv_prep_state_kernel(const float* __restrict__ u, long long ld, int C, int taps, float* __restrict__ state,
                      long long state_stride, long long state_off, const int* __restrict__ cu_tokens,
                      const int* __restrict__ slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
  if (c >= C) return;
  short_conv_advance(u, ld, C, taps, state + (size_t)slots[r] * state_stride + state_off, cu_tokens[r],
                     cu_tokens[r + 1], c);
}

// u float32 [T, ld]; conv_w float32 [H*d + G*d + G*vd, taps] (taps 0: no convolution); state float32 rows
// ``state_stride`` apart with this mixer's (taps - 1) x C kept inputs at ``state_off``, moved on by the portions when
// ``update_state``; norm_mode 0 none, 1 whole projection (wq [H*d], wk [G*d]), 2 per head without weights.
extern "C" int qd_qkv_prep(const float* u, long long ld, int T, int n_requests, int H, int G, int d, int vd, int taps,
                           const float* conv_w, float* state, long long state_stride, long long state_off,
                           const int* token_req, const int* cu_tokens, const int* slots, int update_state,
                           int norm_mode, int norm_after, const float* wq, const float* wk, float eps, int rotary_dim,
                           int pairing, const float* cos_t, const float* sin_t, const int* positions, void* q_out,
                           int q_dtype, void* kv, int kv_dtype, const int* slot_map, int page_size, int write_kv,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long C = (long long)H * d + (long long)G * d + (long long)G * vd;
  if (d <= 0 || d > QP_MAX_D || (d & 1) || vd <= 0 || G <= 0 || H <= 0 || rotary_dim < 0 || rotary_dim > d ||
      (rotary_dim & 1) || taps < 0 || (taps > 1 && !state) || (taps > 0 && !conv_w) || norm_mode < 0 || norm_mode > 2 ||
      (norm_mode == 1 && (!wq || !wk)) || (rotary_dim > 0 && (!cos_t || !sin_t)) || n_requests > 65535)
    return QD_ERR_UNSUPPORTED;
  const size_t smem = ((size_t)C + 40) * sizeof(float);
  if (smem > 200 * 1024) return QD_ERR_UNSUPPORTED;
  static size_t raised = 48 * 1024;
  if (smem > raised) {
    cudaFuncSetAttribute(qkv_prep_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(qkv_prep_kernel<QP_MAX_D / 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    raised = smem;
  }
  // few tokens: a token's channels and heads are shared among more threads (a decode step waits for its longest CTA)
  const int threads = T <= 128 ? (C >= 4096 ? 1024 : 512) : QP_THREADS;
  const int advance = update_state && taps > 1 && T == n_requests;     // single tokens, one per request
  QkvPrep a = {u, ld, H, G, d, vd, taps, conv_w, state, state_stride, state_off, token_req, cu_tokens, slots, advance,
               norm_mode, norm_after, wq, wk, eps, rotary_dim, pairing, cos_t, sin_t, positions, q_out, q_dtype, kv,
               kv_dtype, slot_map, page_size, write_kv};
  if (d <= 128) qd_launch(qkv_prep_kernel<2>, dim3(T), dim3(threads), smem, stream, a);
  else qd_launch(qkv_prep_kernel<QP_MAX_D / 64>, dim3(T), dim3(threads), smem, stream, a);
  if (update_state && taps > 1 && !advance)
    qd_launch(qkv_prep_state_kernel, dim3((unsigned)((C + 255) / 256), n_requests), dim3(256), 0, stream, u, ld, (int)C,
              taps, state, state_stride, state_off, cu_tokens, slots);
  return qd_last_error();
}
