// Grouped-query attention whose softmax has a sink, whose values may have another size than its keys, and whose
// queries and keys are unit-normalised per head before they turn:
//
//   prep      per token: q_h <- unit(q_h) * wq, k_g <- unit(k_g) * wk (unit(y) = y / sqrt(mean(y^2) + eps), over the
//             head; skipped without weights), the first ``rotary_dim`` elements of each turn by the token's
//             position (table rows of cos and sin), v_g <- (1 - lam) v_g + lam v0_g when a source of earlier values
//             is given; q goes to a dense [T, H * d] tensor, k and v to the token's slot of the paged cache
//   attend    p_j = exp(s_j) / (sum_j exp(s_j) + exp(sink_h)) over the keys j <= position (or the last ``window``),
//             s_j = (q . k_j) * scale; the sink has no key and no value.  One warp per (token, head), float32
//             arithmetic, any sizes; tiles of 32 keys counted from key 0, so the order of every sum depends on the
//             token's position only
//
//
// Further options of ``attend`` (``AttnExtra``): ``chunk`` > 0 lets a query see only the keys of its own block of
// ``chunk`` positions (blocks counted from position 0 of the sequence); ``gate`` multiplies head h's output row by
// sigmoid(gate[t * gate_ld + h]) (float32 logits); ``out_scale`` multiplies it by a constant; ``out_stride`` is the
// distance between output rows, so that the heads may land in a column range of a wider tensor.
//
// A page of the cache holds the keys [G, page_size, d] and then the values [G, page_size, vd].
#include "common.cuh"
#include "mma_sync.cuh"
#include <math.h>

#define AS_MAX_D 512
#define AS_WARPS 4

struct AttnExtra {
  int chunk;              // 0: none
  const float* gate;      // float32 logits, row t at t * gate_ld, head h at + h; null: none
  long long gate_ld;
  float out_scale;
  long long out_stride;   // elements between output rows
};

// The first key a query at ``pos`` sees.
__device__ __forceinline__ int as_key_lo(int pos, int window, int chunk) {
  int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) { const int c = pos - pos % chunk; lo = c > lo ? c : lo; }
  return lo;
}
// What the finished row of (token t, head h) is multiplied by.
__device__ __forceinline__ float as_out_factor(const AttnExtra& ex, int t, int h) {
  float f = ex.out_scale;
  if (ex.gate) f *= 1.0f / (1.0f + expf(-ex.gate[(size_t)t * ex.gate_ld + h]));
  return f;
}

__device__ __forceinline__ float as_ld(const void* p, int code, size_t i) {
  return code == QD_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void as_st(void* p, int code, size_t i, float v) {
  if (code == QD_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------------------------------------------------- prep
// One warp per (token, slot): slots 0..H-1 the query heads, H..H+G-1 the key heads, H+G..H+2G-1 the value heads.
// qkv [T, ld]: row = [q (H*d) | k (G*d) | v (G*vd)].
__global__ void __launch_bounds__(AS_WARPS * 32)
qk_norm_rope_write_kernel(const void* __restrict__ qkv, int in_dtype, long long ld, int T, int H, int G, int d, int vd,
                          const float* __restrict__ wq, const float* __restrict__ wk, float eps, int rotary_dim,
                          int pairing, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                          const int* __restrict__ positions, void* __restrict__ q_out, int q_dtype,
                          void* __restrict__ kv, int kv_dtype, const int* __restrict__ slot_map, int page_size,
                          int write_kv, const void* __restrict__ v0, long long v0_ld, const float* __restrict__ lam_p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = H + 2 * G;
  const long long item = (long long)blockIdx.x * AS_WARPS + warp;
  if (item >= (long long)T * slots) return;
  const int t = (int)(item / slots), s = (int)(item - (long long)t * slots);
  const size_t row = (size_t)t * ld;
  const size_t page_elems = (size_t)G * page_size * (d + vd);
  size_t slot = 0, page = 0, off = 0;
  if (s >= H) {
    if (!write_kv) return;
    slot = (size_t)slot_map[t];
    page = slot / page_size;
    off = slot - page * page_size;
  }
  if (s >= H + G) {                                   // a value head
    const int g = s - H - G;
    const size_t src = row + (size_t)H * d + (size_t)G * d + (size_t)g * vd;
    const size_t dst = page * page_elems + (size_t)G * page_size * d + ((size_t)g * page_size + off) * vd;
    const float lam = v0 ? *lam_p : 0.f;
    for (int i = lane; i < vd; i += 32) {
      float v = as_ld(qkv, in_dtype, src + i);
      if (v0) v = (1.0f - lam) * v + lam * as_ld(v0, in_dtype, (size_t)t * v0_ld + (size_t)g * vd + i);
      as_st(kv, kv_dtype, dst + i, v);
    }
    return;
  }
  const bool is_q = s < H;
  const size_t src = row + (is_q ? (size_t)s * d : (size_t)H * d + (size_t)(s - H) * d);
  const float* w = is_q ? wq : wk;
  // pairs (a, b) of the head: pair j = lane + 32 * i holds elements (2j, 2j+1) when the pairing is adjacent, and
  // (j, j + rotary_dim / 2) within the rotated part when it is half-split (elements past the rotated part: adjacent)
  float a[AS_MAX_D / 64], b[AS_MAX_D / 64];
  int ia[AS_MAX_D / 64], ib[AS_MAX_D / 64];
  const int half = rotary_dim / 2, pairs = d / 2;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 64; i++) {
    const int j = lane + 32 * i;
    a[i] = b[i] = 0.f;
    ia[i] = ib[i] = -1;
    if (j < pairs) {
      if (pairing == 1 && j < half) { ia[i] = j; ib[i] = j + half; }
      else { ia[i] = 2 * j; ib[i] = 2 * j + 1; }
      a[i] = as_ld(qkv, in_dtype, src + ia[i]);
      b[i] = as_ld(qkv, in_dtype, src + ib[i]);
      ss = fmaf(a[i], a[i], fmaf(b[i], b[i], ss));
    }
  }
  float last = 0.f;                                   // an odd head size leaves one element without a partner
  if ((d & 1) && lane == 0) { last = as_ld(qkv, in_dtype, src + d - 1); ss = fmaf(last, last, ss); }
  float f = 1.f;
  if (w) f = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
  const int pos = positions[t];
  const size_t dst = is_q ? (size_t)t * H * d + (size_t)s * d
                          : page * page_elems + ((size_t)(s - H) * page_size + off) * d;
  void* out = is_q ? q_out : kv;
  const int oc = is_q ? q_dtype : kv_dtype;
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 64; i++) {
    const int j = lane + 32 * i;
    if (j >= pairs) continue;
    float x = a[i] * f, y = b[i] * f;
    if (w) { x *= w[ia[i]]; y *= w[ib[i]]; }
    if (j < half) {
      const float c = cos_t[(size_t)pos * half + j], sn = sin_t[(size_t)pos * half + j];
      const float xr = x * c - y * sn, yr = y * c + x * sn;
      x = xr; y = yr;
    }
    as_st(out, oc, dst + ia[i], x);
    as_st(out, oc, dst + ib[i], y);
  }
  if ((d & 1) && lane == 0) as_st(out, oc, dst + d - 1, w ? last * f * w[d - 1] : last);
}

extern "C" int qd_qk_norm_rope_write(const void* qkv, int in_dtype, long long ld, int T, int H, int G, int d, int vd,
                                     const float* wq, const float* wk, float eps, int rotary_dim, int pairing,
                                     const float* cos_t, const float* sin_t, const int* positions, void* q_out,
                                     int q_dtype, void* kv, int kv_dtype, const int* slot_map, int page_size,
                                     int write_kv, const void* v0, long long v0_ld, const float* lam,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || d > AS_MAX_D || vd <= 0 || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (!wq) != (!wk))
    return QD_ERR_UNSUPPORTED;
  if (pairing == 1 && (d & 1)) return QD_ERR_UNSUPPORTED;
  const long long items = (long long)T * (H + 2 * G);
  qd_launch(qk_norm_rope_write_kernel, dim3((unsigned)((items + AS_WARPS - 1) / AS_WARPS)), dim3(AS_WARPS * 32), 0,
            stream, qkv, in_dtype, ld, T, H, G, d, vd, wq, wk, eps, rotary_dim, pairing, cos_t, sin_t, positions, q_out,
            q_dtype, kv, kv_dtype, slot_map, page_size, write_kv, v0, v0_ld, lam);
  return qd_last_error();
}

// ----------------------------------------------------------------------------------------------------------- attend
template <typename T>
__global__ void __launch_bounds__(AS_WARPS * 32)
sink_attention_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                              const T* __restrict__ kv, const int* __restrict__ block_table, int max_blocks,
                              const int* __restrict__ token_req, const int* __restrict__ positions, int n_tokens,
                              int H, int G, int d, int vd, int page_size, float scale, int window,
                              const float* __restrict__ sinks, AttnExtra ex) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AS_WARPS + warp;
  if (item >= (long long)n_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const int g = h / (H / G);
  float* qs = smem + (size_t)warp * d;
  const T* qr = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_float(qr[i]);
  __syncwarp();

  const int pos = positions[t];
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  const int key_lo = as_key_lo(pos, window, ex.chunk);
  const size_t page_elems = (size_t)G * page_size * (d + vd);
  const size_t k_head = (size_t)g * page_size * d;
  const size_t v_head = (size_t)G * page_size * d + (size_t)g * page_size * vd;

  float m = -INFINITY, l = 0.0f;
  float o[AS_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 32; i++) o[i] = 0.0f;

  for (int base = key_lo & ~31; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key >= key_lo && key <= pos;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[key / page_size];
      const T* kr = kv + (size_t)page * page_elems + k_head + (size_t)(key % page_size) * d;
      float acc = 0.0f;
      for (int i = 0; i < d; i++) acc = fmaf(qs[i], to_float(kr[i]), acc);
      s = acc * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float c = expf(m - m_new);  // m = -inf on the first tile gives 0
    const float p = valid ? expf(s - m_new) : 0.0f;
    l = l * c + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < AS_MAX_D / 32; i++) o[i] *= c;
    const int jend = pos - base + 1 < 32 ? pos - base + 1 : 32;
    for (int j = 0; j < jend; j++) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      if (kj < key_lo) continue;
      const int page = bt[kj / page_size];
      const T* vr = kv + (size_t)page * page_elems + v_head + (size_t)(kj % page_size) * vd;
#pragma unroll
      for (int i = 0; i < AS_MAX_D / 32; i++) {
        const int idx = lane + 32 * i;
        if (idx < vd) o[i] = fmaf(pj, to_float(vr[idx]), o[i]);
      }
    }
  }
  if (sinks) {                                        // the sink joins the denominator once, unscaled
    const float sk = sinks[h];
    const float m_new = fmaxf(m, sk);
    const float c = expf(m - m_new);
    l = l * c + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < AS_MAX_D / 32; i++) o[i] *= c;
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * vd;
  const float inv = as_out_factor(ex, t, h) / l;
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 32; i++) {
    const int idx = lane + 32 * i;
    if (idx < vd) orow[idx] = from_float<T>(o[i] * inv);
  }
}

// q: first query element, rows q_stride elements apart, head h at h * d; out [n_tokens, H * vd] rows out_stride apart;
// kv: pages of [G, page_size, d] keys then [G, page_size, vd] values; sinks float32 [H] or null.
extern "C" int qd_sink_attention_generic(const void* q, long long q_stride, void* out, long long out_stride,
                                         const void* kv, int dtype, const int* block_table, int max_blocks,
                                         const int* token_req, const int* positions, int n_tokens, int H, int G, int d,
                                         int vd, int page_size, float scale, int window, const float* sinks,
                                         int chunk, const float* gate, long long gate_ld, float out_scale,
                                         cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || d > AS_MAX_D || vd <= 0 || vd > AS_MAX_D || G <= 0 || H % G != 0 || page_size <= 0)
    return QD_ERR_UNSUPPORTED;
  const long long items = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + AS_WARPS - 1) / AS_WARPS);
  const size_t smem = (size_t)AS_WARPS * d * sizeof(float);
  const AttnExtra ex = {chunk, gate, gate_ld, out_scale, out_stride};
  if (dtype == QD_F32)
    qd_launch(sink_attention_generic_kernel<float>, dim3(blocks), dim3(AS_WARPS * 32), smem, stream, (const float*)q,
              q_stride, (float*)out, out_stride, (const float*)kv, block_table, max_blocks, token_req, positions,
              n_tokens, H, G, d, vd, page_size, scale, window, sinks, ex);
  else if (dtype == QD_BF16)
    qd_launch(sink_attention_generic_kernel<bf16>, dim3(blocks), dim3(AS_WARPS * 32), smem, stream, (const bf16*)q,
              q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_table, max_blocks, token_req, positions,
              n_tokens, H, G, d, vd, page_size, scale, window, sinks, ex);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// ------------------------------------------------------------------------------------------------ tensor cores
// The same attention in bfloat16 on mma.sync m16n8k16 (float32 sums), for prompt portions and decoded tokens alike.
// A CTA of four warps owns one tile of 64 rows of one (request, kv head): rows are (token, head within the group)
// pairs, 64 / group tokens of them, so every row reads the same keys and values, which arrive in tiles of 64 keys by
// 16-byte cp.async (two stages) through the block table, key by key: any page size.  Scores stay float32; a softmax
// weight enters P V as TWO bfloat16 numbers (p = hi + lo, two products into one float32 sum), so weights keep 16 bits
// of mantissa.  Head sizes are padded with zero columns in shared memory up to the template's D (keys: 64, 128) and DV
// (values: 64, 96, 128): any multiple of 8 up to 128 runs.  With ``splits`` > 1 the key tiles of a CTA's range are shared among
// gridDim.z CTAs that leave (o, m, l) per row in scratch memory; the CTA that finishes last for a tile (a ticket per
// tile) adds them up with the sink (``sink_combine_kernel`` does, where there are no tickets); with one split the kernel
// finishes the rows itself.
#define TS_ROWS 64
#define TS_KEYS 64
#define TS_PAD 8

template <int D, int DV>
__global__ void __launch_bounds__(128)
sink_attention_mma_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ kv,
                          const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_tokens,
                          const int* __restrict__ start_pos, int n_requests, int H, int G, int d, int vd, int page_size,
                          float scale_log2, int window, const float* __restrict__ sinks, int splits,
                          float* __restrict__ part_o, float* __restrict__ part_ml, int page_shift,
                          unsigned* __restrict__ tickets, int single_tokens, AttnExtra ex) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int KP = D + TS_PAD, VP = DV + TS_PAD;          // row pitches in shared memory (bfloat16)
  extern __shared__ __align__(16) unsigned char ts_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(ts_raw);               // [64][KP]
  bf16* Ks = Qs + TS_ROWS * KP;                             // [2][64][KP]
  bf16* Vs = Ks + 2 * TS_KEYS * KP;                         // [2][64][VP]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int gs = H / G, ntok = TS_ROWS / gs;                // tokens of a tile
  const int g = blockIdx.y, split = blockIdx.z;
  // which request and which of its tiles
  // the grid's first CTAs take the last tiles: with causal keys those stream the most, and they should not be the tail
  int r = 0, b = gridDim.x - 1 - blockIdx.x, len = 0;
  if (single_tokens) {                                      // every request brings one token: tile b is request b
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
  const int tok0 = b * ntok, toks = min(ntok, len - tok0);  // tokens tok0 .. tok0 + toks - 1 of the request's portion
  const int t0 = cu_tokens[r] + tok0, pos0 = start_pos[r] + tok0;
  const int* bt = block_table + (size_t)r * max_blocks;
  const int key_first = as_key_lo(pos0, window, ex.chunk);   // the tile's first token sees the earliest key
  const int key_last = pos0 + toks - 1;
  const int tile_lo = key_first / TS_KEYS, n_tiles_all = key_last / TS_KEYS - tile_lo + 1;
  const int kt_begin = tile_lo + (int)((long long)n_tiles_all * split / splits);
  const int kt_end = tile_lo + (int)((long long)n_tiles_all * (split + 1) / splits);
  const size_t page_elems = (size_t)G * page_size * (d + vd);
  const size_t k_head = (size_t)g * page_size * d, v_head = (size_t)G * page_size * d + (size_t)g * page_size * vd;

  // (page, offset in page) of a key: a shift and a mask where the page size is a power of two
  auto page_of = [&](int kidx, int& off) {
    if (page_shift >= 0) { off = kidx & (page_size - 1); return bt[kidx >> page_shift]; }
    const int lp = kidx / page_size;
    off = kidx - lp * page_size;
    return bt[lp];
  };
  auto fetch = [&](int kt, int stage) {
    bf16* ks = Ks + (size_t)stage * TS_KEYS * KP;
    bf16* vs = Vs + (size_t)stage * TS_KEYS * VP;
    for (int c = tid; c < TS_KEYS * (D / 8); c += 128) {
      const int key = c / (D / 8), col = (c - key * (D / 8)) * 8, kidx = kt * TS_KEYS + key;
      int page = -1, off = 0;
      if (kidx >= key_first && kidx <= key_last && col < d) page = page_of(kidx, off);
      const bf16* src = page >= 0 ? kv + (size_t)page * page_elems + k_head + (size_t)off * d + col : kv;
      ts_cp_async16(ks + key * KP + col, src, page >= 0 ? 16 : 0);
    }
    for (int c = tid; c < TS_KEYS * (DV / 8); c += 128) {
      const int key = c / (DV / 8), col = (c - key * (DV / 8)) * 8, kidx = kt * TS_KEYS + key;
      int page = -1, off = 0;
      if (kidx >= key_first && kidx <= key_last && col < vd) page = page_of(kidx, off);
      const bf16* src = page >= 0 ? kv + (size_t)page * page_elems + v_head + (size_t)off * vd + col : kv;
      ts_cp_async16(vs + key * VP + col, src, page >= 0 ? 16 : 0);
    }
  };

  if (kt_begin < kt_end) fetch(kt_begin, 0);
  ts_commit();
  // the tile's queries: row = token * gs + head within the group; rows past the tile's tokens and columns past d are zero
  for (int c = tid; c < TS_ROWS * (D / 8); c += 128) {
    const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
    const int tk = row / gs, hh = row - tk * gs;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tk < toks && col < d)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(t0 + tk) * H * d + (size_t)(g * gs + hh) * d + col);
    *reinterpret_cast<uint4*>(Qs + row * KP + col) = v;
  }
  __syncthreads();
  unsigned qa[D / 16][4];
  {
    const bf16* q0 = Qs + (warp * 16 + gq) * KP + 2 * tq;
#pragma unroll
    for (int ks = 0; ks < D / 16; ks++) {
      qa[ks][0] = *reinterpret_cast<const unsigned*>(q0 + ks * 16);
      qa[ks][1] = *reinterpret_cast<const unsigned*>(q0 + ks * 16 + 8 * KP);
      qa[ks][2] = *reinterpret_cast<const unsigned*>(q0 + ks * 16 + 8);
      qa[ks][3] = *reinterpret_cast<const unsigned*>(q0 + ks * 16 + 8 * KP + 8);
    }
  }
  // this thread's two rows: r0 = warp * 16 + gq, r1 = r0 + 8
  const int row0 = warp * 16 + gq, row1 = row0 + 8;
  const int tk0 = row0 / gs, tk1 = row1 / gs;
  const bool live0 = tk0 < toks, live1 = tk1 < toks;
  const bool warp_live = warp * 16 < toks * gs;
  const int p0 = pos0 + tk0, p1 = pos0 + tk1;
  const int lo0 = as_key_lo(p0, window, ex.chunk), lo1 = as_key_lo(p1, window, ex.chunk);
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
    const bf16* ks_ = Ks + (size_t)stage * TS_KEYS * KP;
    const bf16* vs_ = Vs + (size_t)stage * TS_KEYS * VP;
    float s[TS_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < TS_KEYS / 8; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    // Two steps of 16 dimensions at a time: one ldmatrix per group of 8 keys fetches both steps' operands, and the
    // eight groups' products follow one another, so that no product waits for the one issued just before it.
#pragma unroll
    for (int ks = 0; ks < D / 16; ks += 2) {
      unsigned kb[TS_KEYS / 8][4];
#pragma unroll
      for (int n = 0; n < TS_KEYS / 8; n++)
        ts_ldmatrix_x4(kb[n], ks_ + (n * 8 + (lane & 7)) * KP + (lane >> 3) * 8 + ks * 16);
#pragma unroll
      for (int n = 0; n < TS_KEYS / 8; n++) ts_mma(s[n], qa[ks], kb[n][0], kb[n][1]);
#pragma unroll
      for (int n = 0; n < TS_KEYS / 8; n++) ts_mma(s[n], qa[ks + 1], kb[n][2], kb[n][3]);
    }
    // mask, scale (scores in units of log 2), row maxima
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < TS_KEYS / 8; n++) {
      const int k0 = kt * TS_KEYS + n * 8 + 2 * tq, k1 = k0 + 1;
      s[n][0] = (live0 && k0 <= p0 && k0 >= lo0) ? s[n][0] * scale_log2 : -INFINITY;
      s[n][1] = (live0 && k1 <= p0 && k1 >= lo0) ? s[n][1] * scale_log2 : -INFINITY;
      s[n][2] = (live1 && k0 <= p1 && k0 >= lo1) ? s[n][2] * scale_log2 : -INFINITY;
      s[n][3] = (live1 && k1 <= p1 && k1 >= lo1) ? s[n][3] * scale_log2 : -INFINITY;
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
    for (int n = 0; n < TS_KEYS / 8; n++) {
      s[n][0] = ts_exp2(s[n][0] - u0); s[n][1] = ts_exp2(s[n][1] - u0);
      s[n][2] = ts_exp2(s[n][2] - u1); s[n][3] = ts_exp2(s[n][3] - u1);
      l0 += s[n][0] + s[n][1];
      l1 += s[n][2] + s[n][3];
    }
    // O += P V, P as hi + lo
#pragma unroll
    for (int j = 0; j < TS_KEYS / 16; j++) {
      unsigned ah[4], al[4];
      ts_split(s[2 * j][0], s[2 * j][1], ah[0], al[0]);
      ts_split(s[2 * j][2], s[2 * j][3], ah[1], al[1]);
      ts_split(s[2 * j + 1][0], s[2 * j + 1][1], ah[2], al[2]);
      ts_split(s[2 * j + 1][2], s[2 * j + 1][3], ah[3], al[3]);
#pragma unroll
      for (int n2 = 0; n2 < DV / 16; n2 += 2) {               // four output groups in flight: a sum is touched again
        unsigned va[4], vb[4];                                // only after three products of other sums
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
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const bool live = half ? live1 : live0;
    if (!live) continue;
    const int row = half ? row1 : row0, tk = half ? tk1 : tk0;
    const int h = g * gs + (row - tk * gs), t = t0 + tk;
    float m = half ? m1 : m0, l = half ? l1 : l0;
    if (splits > 1) {
      const size_t pi = ((size_t)t * H + h) * splits + split;
#pragma unroll
      for (int n = 0; n < DV / 8; n++) {
        const int col = n * 8 + 2 * tq;
        if (col < vd) *reinterpret_cast<float2*>(part_o + pi * vd + col) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
      }
      if (tq == 0) { part_ml[pi * 2] = m; part_ml[pi * 2 + 1] = l; }
      continue;
    }
    float c = 1.f;
    if (sinks) {
      const float sk = sinks[h] * 1.4426950408889634f, mn = fmaxf(m, sk);
      c = exp2f(m - mn);
      l = l * c + exp2f(sk - mn);
    }
    const float f = c / l * as_out_factor(ex, t, h);
#pragma unroll
    for (int n = 0; n < DV / 8; n++) {
      const int col = n * 8 + 2 * tq;
      if (col < vd)
        *reinterpret_cast<unsigned*>(out + (size_t)t * ex.out_stride + (size_t)h * vd + col) =
            ts_pack(o[n][2 * half] * f, o[n][2 * half + 1] * f);
    }
  }
  if (splits == 1 || tickets == nullptr) return;            // without tickets a combine kernel follows
  // The CTA that finishes last for this tile adds up all splits.  Every thread has written its partial results; they
  // meet, then one thread takes the ticket (its fence before the increment releases the CTA's writes, the fence
  // after it acquires the others'), and the reads below go to L2, never to a stale line of this SM's L1.
  __shared__ unsigned s_last;
  __syncthreads();
  if (tid == 0) {
    unsigned* tk = tickets + (size_t)blockIdx.x * G + g;
    __threadfence();
    const unsigned got = atomicAdd(tk, 1u);
    s_last = got == (unsigned)splits - 1;
    if (s_last) *tk = 0;                                    // as found, for the next launch
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  // [rows][splits] the splits' maxima, then their weights in place; [rows][splits] their sums; [rows] 1 / total.
  // Every (row, split) pair is fetched by a thread of its own, in one round of loads; a thread per row then sums up
  // from shared memory.
  float* wgt = reinterpret_cast<float*>(Ks);
  const int rows_live = toks * gs;
  float* sums = wgt + rows_live * splits;
  float* inv_l = sums + rows_live * splits;
  for (int idx = tid; idx < rows_live * splits; idx += 128) {
    const int row = idx / splits, s2 = idx - row * splits;
    const int tk_ = row / gs, h = g * gs + (row - tk_ * gs);
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + ((size_t)(t0 + tk_) * H + h) * splits + s2);
    wgt[idx] = ml.x;
    sums[idx] = ml.y;
  }
  __syncthreads();
  if (tid < rows_live) {
    const int tk_ = tid / gs, h = g * gs + (tid - tk_ * gs);
    const float sk = sinks ? sinks[h] * 1.4426950408889634f : -INFINITY;
    float M = sk;
    for (int s2 = 0; s2 < splits; s2++) M = fmaxf(M, wgt[tid * splits + s2]);
    float L = sinks ? exp2f(sk - M) : 0.f;
    for (int s2 = 0; s2 < splits; s2++) {
      const float m = wgt[tid * splits + s2];
      const float w = m == -INFINITY ? 0.f : exp2f(m - M);
      L += sums[tid * splits + s2] * w;
      wgt[tid * splits + s2] = w;
    }
    inv_l[tid] = as_out_factor(ex, t0 + tk_, h) / L;
  }
  __syncthreads();
  const int vd2 = vd >> 1;                                  // two elements per thread and turn
  for (int idx = tid; idx < rows_live * vd2; idx += 128) {
    const int row = idx / vd2, i = (idx - row * vd2) * 2;
    const int tk_ = row / gs, h = g * gs + (row - tk_ * gs);
    const size_t base = ((size_t)(t0 + tk_) * H + h) * splits;
    float ax = 0.f, ay = 0.f;
#pragma unroll 8
    for (int s2 = 0; s2 < splits; s2++) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(part_o + (base + s2) * vd + i));
      const float w = wgt[row * splits + s2];
      ax = fmaf(v.x, w, ax);
      ay = fmaf(v.y, w, ay);
    }
    const float f = inv_l[row];
    *reinterpret_cast<unsigned*>(out + (size_t)(t0 + tk_) * ex.out_stride + (size_t)h * vd + i) = ts_pack(ax * f, ay * f);
  }
}

// One warp per (token, head): the splits' (o, m, l) and the sink become the output row.  Lane s holds split s's
// maximum and sum (up to 64 splits: two per lane); the output elements then add the splits' rows with weights that
// come by shuffle, so the loads of all splits are independent of one another.
__global__ void __launch_bounds__(128)
sink_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sinks,
                    bf16* __restrict__ out, int n_rows, int H, int vd, int splits, AttnExtra ex) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;                    // t * H + h
  if (row >= n_rows) return;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + (size_t)row * splits;
  const float2 a = lane < splits ? ml[lane] : make_float2(-INFINITY, 0.f);
  const float2 b = lane + 32 < splits ? ml[lane + 32] : make_float2(-INFINITY, 0.f);
  const float sk = sinks ? sinks[row % H] * 1.4426950408889634f : -INFINITY;
  const float M = fmaxf(warp_max(fmaxf(a.x, b.x)), sk);
  const float wa = a.x == -INFINITY ? 0.f : exp2f(a.x - M), wb = b.x == -INFINITY ? 0.f : exp2f(b.x - M);
  const float L = warp_sum(a.y * wa + b.y * wb) + (sinks ? exp2f(sk - M) : 0.f);
  const int t_ = row / H, h_ = row - t_ * H;
  const float inv = as_out_factor(ex, t_, h_) / L;
  const float* po = part_o + (size_t)row * splits * vd;
  for (int i0 = 0; i0 < vd; i0 += 32) {                     // every lane takes every turn: the shuffles need them all
    const int i = i0 + lane;
    float acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; s++) {
      const float w = __shfl_sync(0xffffffffu, s < 32 ? wa : wb, s & 31);
      if (i < vd) acc = fmaf(po[(size_t)s * vd + i], w, acc);
    }
    if (i < vd) out[(size_t)t_ * ex.out_stride + (size_t)h_ * vd + i] = __float2bfloat16_rn(acc * inv);
  }
}

// q [n_tokens, H * d] and out [n_tokens, H * vd] bfloat16, dense; cu_tokens [n_requests + 1] rows of q / out per
// request, start_pos [n_requests] the position of each request's first row; block_table [n_requests, max_blocks].
// tiles: sum over requests of ceil(tokens / (64 / (H / G))) (an upper bound will do).  part_o [n_tokens * H * splits,
// vd] and part_ml [n_tokens * H * splits, 2] float32 when splits > 1.  tickets: tiles * G zeroed words (every launch
// leaves them zero) with which the last CTA of a tile adds up the splits itself; null: a combine kernel follows.
extern "C" int qd_sink_attention_mma(const void* q, void* out, const void* kv, const int* block_table, int max_blocks,
                                     const int* cu_tokens, const int* start_pos, int n_requests, int n_tokens, int tiles,
                                     int H, int G, int d, int vd, int page_size, float scale, int window,
                                     const float* sinks, int splits, float* part_o, float* part_ml,
                                     unsigned* tickets, int chunk, const float* gate, long long gate_ld,
                                     float out_scale, long long out_stride, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return 0;
  if (G <= 0 || H % G || H / G > TS_ROWS || d <= 0 || vd <= 0 || d > 128 || vd > 128 || d % 8 || vd % 8 ||
      page_size <= 0 || splits < 1 || splits > 64 || G > 65535 || (splits > 1 && (!part_o || !part_ml)) ||
      out_stride < (long long)H * vd || (out_stride & 1))
    return QD_ERR_UNSUPPORTED;
  const AttnExtra ex = {chunk, gate, gate_ld, out_scale, out_stride};
  const float scale_log2 = scale * 1.4426950408889634f;
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; page_shift++) {}
  const int single_tokens = n_tokens == n_requests;         // every request has at least one token
  if (single_tokens) tiles = n_requests;
  dim3 grid(tiles, G, splits);
#define TS_GO(D_, DV_)                                                                                              \
  do {                                                                                                              \
    const size_t smem = ((size_t)TS_ROWS * (D_ + TS_PAD) + 2 * TS_KEYS * (D_ + TS_PAD) + 2 * TS_KEYS * (DV_ + TS_PAD)) * 2; \
    static bool raised = false;                                                                                     \
    if (!raised) {                                                                                                  \
      cudaFuncSetAttribute(sink_attention_mma_kernel<D_, DV_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      raised = true;                                                                                                \
    }                                                                                                               \
    qd_launch(sink_attention_mma_kernel<D_, DV_>, grid, dim3(128), smem, stream, (const bf16*)q, (bf16*)out,          \
              (const bf16*)kv, block_table, max_blocks, cu_tokens, start_pos, n_requests, H, G, d, vd, page_size,    \
              scale_log2, window, sinks, splits, part_o, part_ml, page_shift, tickets, single_tokens, ex);           \
  } while (0)
  if (d <= 64 && vd <= 64) TS_GO(64, 64);
  else if (d <= 64) TS_GO(64, 128);
  else if (vd <= 64) TS_GO(128, 64);
  else if (vd <= 96) TS_GO(128, 96);
  else TS_GO(128, 128);
#undef TS_GO
  if (splits > 1 && !tickets) {
    const int rows = n_tokens * H;
    qd_launch(sink_combine_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, (const float*)part_o,
              (const float*)part_ml, sinks, (bf16*)out, rows, H, vd, splits, ex);
  }
  return qd_last_error();
}
