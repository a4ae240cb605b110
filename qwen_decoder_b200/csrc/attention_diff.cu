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
#include "mma_sync.cuh"
#include <math.h>

#define AD_MAX_VD 512
#define AD_WARPS 4

// ------------------------------------------------------------------------------------------------------------- prep
// One thread per (token, channel) of the first ``C`` = Cq + Ck + Cv columns of u.
template <typename TC>
__global__ void __launch_bounds__(256)
diff_conv_write_kernel(const float* __restrict__ u, long long ldu, int Cq, int Ck, int Cv, int taps,
                       const float* __restrict__ w, float* state, long long state_stride,
                       long long state_off, const int* __restrict__ token_req, const int* __restrict__ cu_tokens,
                       const int* __restrict__ slots, TC* __restrict__ q_out, TC* __restrict__ kv,
                       const int* __restrict__ slot_map, int page_size, int G, int d2, int vd, int write_kv,
                       int advance) {
  pdl_launch_dependents();
  pdl_wait();
  const int C = Cq + Ck + Cv;
  const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
  if (c >= C) return;
  if (c >= Cq && !write_kv) return;
  float y;
  if (taps > 0) {
    const int r = token_req[t];
    float* st = state ? state + (size_t)slots[r] * state_stride + state_off : nullptr;
    y = short_conv_at(u, ldu, C, taps, w, st, cu_tokens[r], t, c);
    // every request brings one token: this thread alone reads and writes channel c of its request's kept inputs
    if (advance) short_conv_advance(u, ldu, C, taps, st, t, t + 1, c);
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
  // single tokens (one per request): the convolution's own launch moves the kept inputs on
  const int advance = write && taps > 1 && T == n_requests;
  if (dtype == QD_F32)
    qd_launch(diff_conv_write_kernel<float>, grid, dim3(256), 0, stream, u, ldu, Cq, Ck, Cv, taps, w,
              state, state_stride, state_off, token_req, cu_tokens, slots, (float*)q_out, (float*)kv,
              slot_map, page_size, G, d2, vd, write, advance);
  else if (dtype == QD_BF16)
    qd_launch(diff_conv_write_kernel<bf16>, grid, dim3(256), 0, stream, u, ldu, Cq, Ck, Cv, taps, w,
              state, state_stride, state_off, token_req, cu_tokens, slots, (bf16*)q_out, (bf16*)kv,
              slot_map, page_size, G, d2, vd, write, advance);
  else
    return QD_ERR_UNSUPPORTED;
  if (write && taps > 1 && !advance)
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

// ------------------------------------------------------------------------------------------- attend, tensor cores
// The same attention in bfloat16 on mma.sync m16n8k16 (float32 sums), for prompt portions and decoded tokens alike.
// A CTA of four warps owns one tile of one (request, kv head): 32 (token, head within the group) pairs, each as TWO
// rows, one per map.  Warps 0 and 1 hold the pairs' first maps, warps 2 and 3 their second maps: a warp's 16 rows
// all read the same half of a key row (columns [map * d, map * d + d)) and the same values, so each warp is an
// ordinary attention over 64-key tiles (16-byte cp.async, two stages, key by key through the block table: any page
// size).  Scores, the cap and the softmax stay float32; a weight enters P V as two bfloat16 numbers (hi + lo).  Head
// sizes are padded with zero columns in shared memory up to the template's D (64, 128) and DV (64, 128).
// With one split the two maps of a pair meet in shared memory at the end, where the difference, its unit norm, the
// constant and the gate are applied; with ``splits`` > 1 the key tiles are shared among gridDim.z CTAs that leave
// (o, m, l) per (row, map) in scratch memory, and ``diff_combine_kernel`` finishes.
#define DM_PAIRS 32
#define DM_KEYS 64
#define DM_PAD 8
#define DM_LOG2E 1.4426950408889634f

// a score in units of log 2: raw * scale, capped when a cap is given.  tanh(x) = 1 - 2 / (e^(2x) + 1): the absolute
// error stays near 1e-7 for every x (large x: e^(2x) = inf, 2 / inf = 0).
__device__ __forceinline__ float dm_score(float raw, float k_in, float k_out, bool capped) {
  if (!capped) return raw * k_in;                           // k_in = scale * log2(e)
  const float e = ts_exp2(raw * k_in);                      // k_in = 2 * log2(e) * scale / cap
  return (1.0f - __fdividef(2.0f, e + 1.0f)) * k_out;       // k_out = cap * log2(e)
}

template <int D, int DV>
__global__ void __launch_bounds__(128)
diff_attention_mma_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ kv,
                          const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_tokens,
                          const int* __restrict__ start_pos, int n_requests, int H, int G, int d, int vd, int page_size,
                          DiffParams P, int window, int splits, float* __restrict__ part_o,
                          float* __restrict__ part_ml, int page_shift, int single_tokens,
                          const float* __restrict__ gate, long long ldg) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int QP = D + DM_PAD, KP = 2 * D + DM_PAD, VP = DV + DM_PAD;   // row pitches in shared memory (bfloat16)
  constexpr int FP = DV + 4;                                               // pitch of the float32 rows at the end
  extern __shared__ __align__(16) unsigned char dm_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(dm_raw);               // [2 maps][32 pairs][QP]
  bf16* Ks = Qs + 2 * DM_PAIRS * QP;                        // [2 stages][64][KP]: a key row is [map 1 (D) | map 2 (D)]
  bf16* Vs = Ks + 2 * DM_KEYS * KP;                         // [2 stages][64][VP]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int map = warp >> 1;
  const int gs = H / G, ntok = DM_PAIRS / gs;               // tokens of a tile
  const int g = blockIdx.y, split = blockIdx.z;
  const int d2 = 2 * d;
  int r = 0, b = gridDim.x - 1 - blockIdx.x, len = 0;       // the grid's first CTAs take the last (longest) tiles
  if (single_tokens) {
    r = b;
    b = 0;
    len = 1;
  } else {
    for (; r < n_requests; r++) {
      len = cu_tokens[r + 1] - cu_tokens[r];
      const int tiles = (len + ntok - 1) / ntok;
      if (b < tiles) break;
      b -= tiles;
    }
  }
  if (r >= n_requests) return;
  const int tok0 = b * ntok, toks = min(ntok, len - tok0);
  const int t0 = cu_tokens[r] + tok0, pos0 = start_pos[r] + tok0;
  const int* bt = block_table + (size_t)r * max_blocks;
  const int key_first = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int key_last = pos0 + toks - 1;
  const int tile_lo = key_first / DM_KEYS, n_tiles_all = key_last / DM_KEYS - tile_lo + 1;
  const int kt_begin = tile_lo + (int)((long long)n_tiles_all * split / splits);
  const int kt_end = tile_lo + (int)((long long)n_tiles_all * (split + 1) / splits);
  const size_t page_elems = (size_t)G * page_size * (d2 + vd);
  const size_t k_head = (size_t)g * page_size * d2, v_head = (size_t)G * page_size * d2 + (size_t)g * page_size * vd;

  auto page_of = [&](int kidx, int& off) {
    if (page_shift >= 0) { off = kidx & (page_size - 1); return bt[kidx >> page_shift]; }
    const int lp = kidx / page_size;
    off = kidx - lp * page_size;
    return bt[lp];
  };
  auto fetch = [&](int kt, int stage) {
    bf16* ks = Ks + (size_t)stage * DM_KEYS * KP;
    bf16* vs = Vs + (size_t)stage * DM_KEYS * VP;
    for (int c = tid; c < DM_KEYS * (2 * D / 8); c += 128) {
      const int key = c / (2 * D / 8), pc = (c - key * (2 * D / 8)) * 8, kidx = kt * DM_KEYS + key;
      const int mp = pc >= D, col = pc - mp * D;            // padded column pc = map mp's column col
      int page = -1, off = 0;
      if (kidx >= key_first && kidx <= key_last && col < d) page = page_of(kidx, off);
      const bf16* src = page >= 0 ? kv + (size_t)page * page_elems + k_head + (size_t)off * d2 + mp * d + col : kv;
      ts_cp_async16(ks + key * KP + pc, src, page >= 0 ? 16 : 0);
    }
    for (int c = tid; c < DM_KEYS * (DV / 8); c += 128) {
      const int key = c / (DV / 8), col = (c - key * (DV / 8)) * 8, kidx = kt * DM_KEYS + key;
      int page = -1, off = 0;
      if (kidx >= key_first && kidx <= key_last && col < vd) page = page_of(kidx, off);
      const bf16* src = page >= 0 ? kv + (size_t)page * page_elems + v_head + (size_t)off * vd + col : kv;
      ts_cp_async16(vs + key * VP + col, src, page >= 0 ? 16 : 0);
    }
  };

  if (kt_begin < kt_end) fetch(kt_begin, 0);
  ts_commit();
  // the tile's queries: row = map * 32 + pair, pair = token * gs + head within the group; the rest is zero
  for (int c = tid; c < 2 * DM_PAIRS * (D / 8); c += 128) {
    const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
    const int mp = row / DM_PAIRS, pr = row - mp * DM_PAIRS;
    const int tk = pr / gs, hh = pr - tk * gs;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tk < toks && col < d)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(t0 + tk) * H * d2 + (size_t)(g * gs + hh) * d2 + mp * d + col);
    *reinterpret_cast<uint4*>(Qs + row * QP + col) = v;
  }
  __syncthreads();
  unsigned qa[D / 16][4];
  {
    const bf16* q0 = Qs + (warp * 16 + gq) * QP + 2 * tq;
#pragma unroll
    for (int ks = 0; ks < D / 16; ks++) {
      qa[ks][0] = *reinterpret_cast<const unsigned*>(q0 + ks * 16);
      qa[ks][1] = *reinterpret_cast<const unsigned*>(q0 + ks * 16 + 8 * QP);
      qa[ks][2] = *reinterpret_cast<const unsigned*>(q0 + ks * 16 + 8);
      qa[ks][3] = *reinterpret_cast<const unsigned*>(q0 + ks * 16 + 8 * QP + 8);
    }
  }
  // this thread's two rows are the pairs pr0 and pr0 + 8 of its warp's map
  const int pr0 = (warp & 1) * 16 + gq, pr1 = pr0 + 8;
  const int tk0 = pr0 / gs, tk1 = pr1 / gs;
  const bool live0 = tk0 < toks, live1 = tk1 < toks;
  const bool warp_live = (warp & 1) * 16 < toks * gs;
  const int p0 = pos0 + tk0, p1 = pos0 + tk1;
  const int lo0 = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
  const int lo1 = (window > 0 && p1 - window + 1 > 0) ? p1 - window + 1 : 0;
  const bool capped = P.cap > 0.f;
  const float k_in = capped ? 2.0f * DM_LOG2E * P.scale / P.cap : P.scale * DM_LOG2E;
  const float k_out = P.cap * DM_LOG2E;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int kt = kt_begin; kt < kt_end; kt++) {
    const int stage = (kt - kt_begin) & 1;
    if (kt + 1 < kt_end) fetch(kt + 1, stage ^ 1);
    ts_commit();
    ts_wait<1>();
    __syncthreads();
    if (!warp_live) { __syncthreads(); continue; }          // this warp's 16 rows hold no token: it only fetches
    const bf16* ks_ = Ks + (size_t)stage * DM_KEYS * KP + map * D;
    const bf16* vs_ = Vs + (size_t)stage * DM_KEYS * VP;
    float s[DM_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < DM_KEYS / 8; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ks += 2) {
      unsigned kb[DM_KEYS / 8][4];
#pragma unroll
      for (int n = 0; n < DM_KEYS / 8; n++)
        ts_ldmatrix_x4(kb[n], ks_ + (n * 8 + (lane & 7)) * KP + (lane >> 3) * 8 + ks * 16);
#pragma unroll
      for (int n = 0; n < DM_KEYS / 8; n++) ts_mma(s[n], qa[ks], kb[n][0], kb[n][1]);
#pragma unroll
      for (int n = 0; n < DM_KEYS / 8; n++) ts_mma(s[n], qa[ks + 1], kb[n][2], kb[n][3]);
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < DM_KEYS / 8; n++) {
      const int k0 = kt * DM_KEYS + n * 8 + 2 * tq, k1 = k0 + 1;
      s[n][0] = (live0 && k0 <= p0 && k0 >= lo0) ? dm_score(s[n][0], k_in, k_out, capped) : -INFINITY;
      s[n][1] = (live0 && k1 <= p0 && k1 >= lo0) ? dm_score(s[n][1], k_in, k_out, capped) : -INFINITY;
      s[n][2] = (live1 && k0 <= p1 && k0 >= lo1) ? dm_score(s[n][2], k_in, k_out, capped) : -INFINITY;
      s[n][3] = (live1 && k1 <= p1 && k1 >= lo1) ? dm_score(s[n][3], k_in, k_out, capped) : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
      mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
    }
    const float mn0 = fmaxf(m0, ts_quad_max(mx0)), mn1 = fmaxf(m1, ts_quad_max(mx1));
    const float u0 = mn0 == -INFINITY ? 0.f : mn0, u1 = mn1 == -INFINITY ? 0.f : mn1;   // a row with no key yet
    const float c0 = ts_exp2(m0 - u0), c1 = ts_exp2(m1 - u1);
    m0 = mn0; m1 = mn1;
    l0 *= c0; l1 *= c1;
#pragma unroll
    for (int n = 0; n < DV / 8; n++) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
#pragma unroll
    for (int n = 0; n < DM_KEYS / 8; n++) {
      s[n][0] = ts_exp2(s[n][0] - u0); s[n][1] = ts_exp2(s[n][1] - u0);
      s[n][2] = ts_exp2(s[n][2] - u1); s[n][3] = ts_exp2(s[n][3] - u1);
      l0 += s[n][0] + s[n][1];
      l1 += s[n][2] + s[n][3];
    }
#pragma unroll
    for (int j = 0; j < DM_KEYS / 16; j++) {
      unsigned ah[4], al[4];
      ts_split(s[2 * j][0], s[2 * j][1], ah[0], al[0]);
      ts_split(s[2 * j][2], s[2 * j][3], ah[1], al[1]);
      ts_split(s[2 * j + 1][0], s[2 * j + 1][1], ah[2], al[2]);
      ts_split(s[2 * j + 1][2], s[2 * j + 1][3], ah[3], al[3]);
#pragma unroll
      for (int n2 = 0; n2 < DV / 16; n2 += 2) {
        unsigned va[4], vb[4];
        ts_ldmatrix_x4_trans(va, vs_ + (j * 16 + (lane & 15)) * VP + n2 * 16 + (lane >> 4) * 8);
        ts_ldmatrix_x4_trans(vb, vs_ + (j * 16 + (lane & 15)) * VP + (n2 + 1) * 16 + (lane >> 4) * 8);
        ts_mma(o[2 * n2], ah, va[0], va[1]);
        ts_mma(o[2 * n2 + 1], ah, va[2], va[3]);
        ts_mma(o[2 * n2 + 2], ah, vb[0], vb[1]);
        ts_mma(o[2 * n2 + 3], ah, vb[2], vb[3]);
        ts_mma(o[2 * n2], al, va[0], va[1]);
        ts_mma(o[2 * n2 + 1], al, va[2], va[3]);
        ts_mma(o[2 * n2 + 2], al, vb[0], vb[1]);
        ts_mma(o[2 * n2 + 3], al, vb[2], vb[3]);
      }
    }
    __syncthreads();          // all warps are done with this stage before the next fetch overwrites it
  }
  ts_wait<0>();
  l0 = ts_quad_sum(l0);
  l1 = ts_quad_sum(l1);
  if (splits > 1) {
#pragma unroll
    for (int half = 0; half < 2; half++) {
      if (!(half ? live1 : live0)) continue;
      const int pr = half ? pr1 : pr0, tk = half ? tk1 : tk0;
      const int h = g * gs + (pr - tk * gs), t = t0 + tk;
      const size_t pi = (((size_t)t * H + h) * 2 + map) * splits + split;
#pragma unroll
      for (int n = 0; n < DV / 8; n++) {
        const int col = n * 8 + 2 * tq;
        if (col < vd) *reinterpret_cast<float2*>(part_o + pi * vd + col) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
      }
      if (tq == 0) { part_ml[pi * 2] = half ? m1 : m0; part_ml[pi * 2 + 1] = half ? l1 : l0; }
    }
    return;
  }
  // one split: both maps of a pair meet in shared memory (the key and value stages are free now)
  __syncthreads();
  float* F = reinterpret_cast<float*>(Ks);                  // [2 maps][32 pairs][FP]
#pragma unroll
  for (int half = 0; half < 2; half++) {
    if (!(half ? live1 : live0)) continue;
    const int pr = half ? pr1 : pr0;
    const float inv = 1.0f / (half ? l1 : l0);
    float* fr = F + (size_t)(map * DM_PAIRS + pr) * FP;
#pragma unroll
    for (int n = 0; n < DV / 8; n++)
      *reinterpret_cast<float2*>(fr + n * 8 + 2 * tq) = make_float2(o[n][2 * half] * inv, o[n][2 * half + 1] * inv);
  }
  __syncthreads();
  for (int pr = warp; pr < toks * gs; pr += 4) {
    const int tk = pr / gs, h = g * gs + (pr - tk * gs), t = t0 + tk;
    const float* f1 = F + (size_t)pr * FP;
    const float* f2 = F + (size_t)(DM_PAIRS + pr) * FP;
    float a[DV / 32], ss = 0.f;
#pragma unroll
    for (int i = 0; i < DV / 32; i++) {
      const int idx = lane + 32 * i;
      a[i] = idx < vd ? f1[idx] - P.lambda * f2[idx] : 0.f;
      ss = fmaf(a[i], a[i], ss);
    }
    ss = warp_sum(ss);
    float f = P.out_scale / sqrtf(ss / (float)vd + P.eps);
    if (gate) f /= 1.0f + expf(-gate[(size_t)t * ldg + h]);
    bf16* orow = out + ((size_t)t * H + h) * vd;
#pragma unroll
    for (int i = 0; i < DV / 32; i++) {
      const int idx = lane + 32 * i;
      if (idx < vd) orow[idx] = __float2bfloat16_rn(a[i] * f);
    }
  }
}

// One CTA of 128 threads per (token, head): the splits' (o, m, l) of both maps become the output row.  Warp m makes map
// m's weights (lane s holds split s's maximum and sum; up to 64 splits, two per lane); thread i then adds element i of
// all splits' rows, loads that do not depend on one another, and the block's sum of squares gives the unit norm.
// vd <= 128.
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                    int n_rows, int H, int vd, int splits, DiffParams P, const float* __restrict__ gate,
                    long long ldg) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float wgt[2][64];
  __shared__ float inv_l[2];
  __shared__ float scratch[40];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.x;                               // t * H + h
  const size_t base = (size_t)row * 2 * splits;
  if (warp < 2) {
    const float2* ml = reinterpret_cast<const float2*>(part_ml) + base + (size_t)warp * splits;
    const float2 x = lane < splits ? ml[lane] : make_float2(-INFINITY, 0.f);
    const float2 y = lane + 32 < splits ? ml[lane + 32] : make_float2(-INFINITY, 0.f);
    const float M = warp_max(fmaxf(x.x, y.x));
    const float wx = x.x == -INFINITY ? 0.f : exp2f(x.x - M), wy = y.x == -INFINITY ? 0.f : exp2f(y.x - M);
    const float L = warp_sum(x.y * wx + y.y * wy);
    wgt[warp][lane] = wx;
    wgt[warp][lane + 32] = wy;
    if (lane == 0) inv_l[warp] = 1.0f / L;
  }
  __syncthreads();
  float a1 = 0.f, a2 = 0.f;
  if (tid < vd) {
    const float* p1 = part_o + base * vd + tid;
    const float* p2 = p1 + (size_t)splits * vd;
#pragma unroll 8
    for (int s = 0; s < splits; s++) {
      a1 = fmaf(p1[(size_t)s * vd], wgt[0][s], a1);
      a2 = fmaf(p2[(size_t)s * vd], wgt[1][s], a2);
    }
  }
  const float o = tid < vd ? a1 * inv_l[0] - P.lambda * (a2 * inv_l[1]) : 0.f;
  const float ss = block_sum(o * o, scratch);
  float f = P.out_scale / sqrtf(ss / (float)vd + P.eps);
  if (gate) f /= 1.0f + expf(-gate[(size_t)(row / H) * ldg + row % H]);
  if (tid < vd) out[(size_t)row * vd + tid] = __float2bfloat16_rn(o * f);
}

// q [n_tokens, H * 2d] and out [n_tokens, H * vd] bfloat16, dense; cu_tokens [n_requests + 1] rows of q / out per
// request, start_pos [n_requests] the position of each request's first row; block_table [n_requests, max_blocks].
// tiles: an upper bound of the sum over requests of ceil(tokens / (32 / (H / G))).  part_o [n_tokens * H * 2 * splits,
// vd] and part_ml [n_tokens * H * 2 * splits, 2] float32 when splits > 1.  gate as in the generic kernel.
extern "C" int qd_diff_attention_mma(const void* q, void* out, const void* kv, const int* block_table, int max_blocks,
                                     const int* cu_tokens, const int* start_pos, int n_requests, int n_tokens,
                                     int tiles, int H, int G, int d, int vd, int page_size, float scale, float cap,
                                     float lambda, float eps, float out_scale, int window, const float* gate,
                                     long long ldg, int splits, float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return 0;
  if (G <= 0 || H % G || H / G > DM_PAIRS || d <= 0 || vd <= 0 || d > 128 || vd > 128 || d % 8 || vd % 8 ||
      page_size <= 0 || splits < 1 || splits > 64 || G > 65535 || (splits > 1 && (!part_o || !part_ml)))
    return QD_ERR_UNSUPPORTED;
  const DiffParams P = {scale, cap, lambda, eps, out_scale};
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; page_shift++) {}
  const int single_tokens = n_tokens == n_requests;         // every request has at least one token
  if (single_tokens) tiles = n_requests;
  dim3 grid(tiles, G, splits);
#define DM_GO(D_, DV_)                                                                                              \
  do {                                                                                                              \
    const size_t smem = ((size_t)2 * DM_PAIRS * (D_ + DM_PAD) + 2 * DM_KEYS * (2 * D_ + DM_PAD) +                   \
                         2 * DM_KEYS * (DV_ + DM_PAD)) * 2;                                                         \
    static bool raised = false;                                                                                     \
    if (!raised) {                                                                                                  \
      cudaFuncSetAttribute(diff_attention_mma_kernel<D_, DV_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      raised = true;                                                                                                \
    }                                                                                                               \
    qd_launch(diff_attention_mma_kernel<D_, DV_>, grid, dim3(128), smem, stream, (const bf16*)q, (bf16*)out,        \
              (const bf16*)kv, block_table, max_blocks, cu_tokens, start_pos, n_requests, H, G, d, vd, page_size, P, \
              window, splits, part_o, part_ml, page_shift, single_tokens, gate, ldg);                               \
  } while (0)
  if (d <= 64 && vd <= 64) DM_GO(64, 64);
  else if (d <= 64) DM_GO(64, 128);
  else if (vd <= 64) DM_GO(128, 64);
  else DM_GO(128, 128);
#undef DM_GO
  if (splits > 1) {
    const int rows = n_tokens * H;
    qd_launch(diff_combine_kernel, dim3(rows), dim3(128), 0, stream, (const float*)part_o,
              (const float*)part_ml, (bf16*)out, rows, H, vd, splits, P, gate, ldg);
  }
  return qd_last_error();
}
