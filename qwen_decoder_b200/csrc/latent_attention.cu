// Latent attention: keys and values of all heads are expanded from ONE cached row per token,
//   row_j = [ c_j (kv_rank, RMS-normed latent) | kr_j (rot_dim, rotated key part shared by the heads) ],
// with k_h,j = Wuk_h c_j and v_h,j = Wuv_h c_j.  The kernels never expand them: since
//   q_h . (Wuk_h c_j) = (Wuk_h^T q_h) . c_j   and   sum_j p_j (Wuv_h c_j) = Wuv_h (sum_j p_j c_j),
// a query is first carried into the latent space (``absorb``), attention runs over the cached rows
// themselves -- every head of a token reads the same rows, so a CTA stages a tile of rows once for
// all its heads -- and the result is carried out of the latent space afterwards (``expand``).
//
//   prep     RMS norms of the query latent and of c (float32), rotation of kr, write of the cache row
//   absorb   qcat[t, h] = [ Wuk_h^T qn[t, h] | rotate(qr[t, h]) ]                    float32
//   attend   o_lat[t, h] = softmax_j<=pos(qcat[t, h] . row_j * scale) c_j            float32, paged, split over keys
//   combine  the splits' partial results into o_lat
//   expand   out[t, h] = (Wuv_h o_lat[t, h]) * sigmoid(gate[t, h])
//
// Scores, softmax weights, norms and angles are float32 in both engine dtypes; the cache row and the
// weights are the engine's dtype.  One template serves float32 and bfloat16.
#include "common.cuh"

// 16 bytes of a row as floats (8 bfloat16 or 4 float32)
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) { float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  __device__ static void load(const bf16* p, float* o) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) { o[2 * i] = __low2float(h[i]); o[2 * i + 1] = __high2float(h[i]); }
  }
};

#define LA_WARPS 8
#define LA_TILE 32          // keys per staged tile
#define LA_MAX_R 512        // latent size the attend kernel takes (16 accumulators a lane)
#define LA_TT 8             // tokens per CTA in absorb and expand

// ----------------------------------------------------------------------------- prep
// u row t (float32, stride ldu): columns [q_off, q_off + q_rank) the raw query latent (q_rank 0: the design has
// none, its queries are a projection of the input itself), [kv_off, kv_off + r + dr) the raw key/value latent
// followed by the key part that is rotated (dr 0: no such part).
template <typename TC>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const float* __restrict__ u, long long ldu, int q_off, int q_rank, int kv_off, int r, int dr,
                   const float* __restrict__ wq_norm, const float* __restrict__ wkv_norm, float eps,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                   const int* __restrict__ positions, const int* __restrict__ slot_map, TC* __restrict__ cq,
                   TC* __restrict__ cache, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[40];
  const int t = blockIdx.x;
  const float* row = u + (size_t)t * ldu;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { float v = row[q_off + i]; sq = fmaf(v, v, sq); }
  for (int i = threadIdx.x; i < r; i += blockDim.x) { float v = row[kv_off + i]; sk = fmaf(v, v, sk); }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  const float iq = q_rank > 0 ? 1.0f / sqrtf(sq / (float)q_rank + eps) : 0.f;      // no query latent: nothing to norm
  const float ik = 1.0f / sqrtf(sk / (float)r + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)t * q_rank + i] = from_float<TC>(row[q_off + i] * iq * wq_norm[i]);
  if (!write_cache) return;
  TC* dst = cache + (size_t)slot_map[t] * (r + dr);
  for (int i = threadIdx.x; i < r; i += blockDim.x) dst[i] = from_float<TC>(row[kv_off + i] * ik * wkv_norm[i]);
  const int pos = positions[t];
  const int half = rot_dims >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
    float a = row[kv_off + r + 2 * i], b = row[kv_off + r + 2 * i + 1];
    dst[r + 2 * i] = from_float<TC>(a * c - b * s);
    dst[r + 2 * i + 1] = from_float<TC>(b * c + a * s);
  }
  for (int i = rot_dims + threadIdx.x; i < dr; i += blockDim.x) dst[r + i] = from_float<TC>(row[kv_off + r + i]);
}

// ----------------------------------------------------------------------------- absorb
// q [T, H * (dn + dr)] float32, rows ldq apart; Wuk [H * dn, r]; qcat [T, H, r + dr] float32.
template <typename TW>
__global__ void __launch_bounds__(256)
latent_absorb_kernel(const float* __restrict__ q, long long ldq, const TW* __restrict__ wuk, float* __restrict__ qcat,
                     int T, int H, int dn, int dr, int r, const float* __restrict__ cos_t,
                     const float* __restrict__ sin_t, int rot_dims, const int* __restrict__ positions,
                     const float* __restrict__ pre) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float qs[];                // [LA_TT][dn]
  const int h = blockIdx.y, t0 = blockIdx.x * LA_TT;
  const int nt = min(LA_TT, T - t0);
  const int W = r + dr;
  const size_t qw = (size_t)ldq;              // q's rows are ldq floats apart (a column range of a wider buffer is fine)
  for (int i = threadIdx.x; i < LA_TT * dn; i += blockDim.x) {
    int tt = i / dn, d = i - tt * dn;
    qs[i] = tt < nt ? q[(size_t)(t0 + tt) * qw + (size_t)h * (dn + dr) + d] : 0.f;
  }
  __syncthreads();
  for (int j = blockIdx.z * blockDim.x + threadIdx.x; j < r; j += gridDim.z * blockDim.x) {
    if (pre) {          // the products were made elsewhere ([H, T, r]): only their place changes
      for (int tt = 0; tt < nt; tt++)
        qcat[((size_t)(t0 + tt) * H + h) * W + j] = pre[((size_t)h * T + t0 + tt) * r + j];
      continue;
    }
    float acc[LA_TT];
#pragma unroll
    for (int tt = 0; tt < LA_TT; tt++) acc[tt] = 0.f;
    const TW* wcol = wuk + (size_t)h * dn * r + j;
    for (int d = 0; d < dn; d++) {
      float w = to_float(wcol[(size_t)d * r]);
#pragma unroll
      for (int tt = 0; tt < LA_TT; tt++) acc[tt] = fmaf(qs[tt * dn + d], w, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < LA_TT; tt++)
      if (tt < nt) qcat[((size_t)(t0 + tt) * H + h) * W + j] = acc[tt];
  }
  if (blockIdx.z != 0) return;
  const int half = rot_dims >> 1;
  for (int i = threadIdx.x; i < nt * dr; i += blockDim.x) {
    int tt = i / dr, e = i - tt * dr;
    const float* qr = q + (size_t)(t0 + tt) * qw + (size_t)h * (dn + dr) + dn;
    float v;
    if (e < rot_dims) {
      int pr = e >> 1, pos = positions[t0 + tt];
      float c = cos_t[(size_t)pos * half + pr], s = sin_t[(size_t)pos * half + pr];
      float a = qr[2 * pr], b = qr[2 * pr + 1];
      v = (e & 1) ? b * c + a * s : a * c - b * s;
    } else {
      v = qr[e];
    }
    qcat[((size_t)(t0 + tt) * H + h) * W + r + e] = v;
  }
}

// The same with 16-byte loads of Wuk, for latent sizes whose pieces divide the CTA evenly (r / V a divisor of 256):
// thread (jg, dg) owns V consecutive latent columns and every (256 * V / r)-th unrotated dimension; the groups'
// partial sums meet in shared memory.  grid (token tiles, heads).
template <typename TW>
__global__ void __launch_bounds__(256)
latent_absorb_vec_kernel(const float* __restrict__ q, long long ldq, const TW* __restrict__ wuk,
                         float* __restrict__ qcat, int T, int H, int dn, int dr, int r,
                         const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                         const int* __restrict__ positions) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = Vec16<TW>::N;
  extern __shared__ float sm[];
  float* qs = sm;                              // [LA_TT][dn]
  float* red = sm + LA_TT * dn;                // [LA_TT][r]
  const int h = blockIdx.y, t0 = blockIdx.x * LA_TT;
  const int nt = min(LA_TT, T - t0);
  const int W = r + dr;
  const size_t qw = (size_t)ldq;              // q's rows are ldq floats apart (a column range of a wider buffer is fine)
  for (int i = threadIdx.x; i < LA_TT * dn; i += blockDim.x) {
    int tt = i / dn, d = i - tt * dn;
    qs[i] = tt < nt ? q[(size_t)(t0 + tt) * qw + (size_t)h * (dn + dr) + d] : 0.f;
  }
  for (int i = threadIdx.x; i < LA_TT * r; i += blockDim.x) red[i] = 0.f;
  __syncthreads();
  const int JG = r / V, DG = 256 / JG;
  const int jg = threadIdx.x % JG, dg = threadIdx.x / JG;
  float acc[LA_TT][V];
#pragma unroll
  for (int tt = 0; tt < LA_TT; tt++)
#pragma unroll
    for (int v = 0; v < V; v++) acc[tt][v] = 0.f;
  const TW* wbase = wuk + (size_t)h * dn * r + jg * V;
#pragma unroll 4
  for (int d = dg; d < dn; d += DG) {
    float w[V];
    Vec16<TW>::load(wbase + (size_t)d * r, w);
#pragma unroll
    for (int tt = 0; tt < LA_TT; tt++) {
      const float qv = qs[tt * dn + d];
#pragma unroll
      for (int v = 0; v < V; v++) acc[tt][v] = fmaf(qv, w[v], acc[tt][v]);
    }
  }
  for (int turn = 0; turn < DG; turn++) {        // the groups add in turn: the order of additions is fixed
    if (dg == turn) {
#pragma unroll
      for (int tt = 0; tt < LA_TT; tt++)
#pragma unroll
        for (int v = 0; v < V; v++) red[tt * r + jg * V + v] += acc[tt][v];
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < nt * r; i += blockDim.x) {
    int tt = i / r, j = i - tt * r;
    qcat[((size_t)(t0 + tt) * H + h) * W + j] = red[i];
  }
  const int half = rot_dims >> 1;
  for (int i = threadIdx.x; i < nt * dr; i += blockDim.x) {
    int tt = i / dr, e = i - tt * dr;
    const float* qr = q + (size_t)(t0 + tt) * qw + (size_t)h * (dn + dr) + dn;
    float v;
    if (e < rot_dims) {
      int pr = e >> 1, pos = positions[t0 + tt];
      float c = cos_t[(size_t)pos * half + pr], sn = sin_t[(size_t)pos * half + pr];
      float a = qr[2 * pr], b = qr[2 * pr + 1];
      v = (e & 1) ? b * c + a * sn : a * c - b * sn;
    } else {
      v = qr[e];
    }
    qcat[((size_t)(t0 + tt) * H + h) * W + r + e] = v;
  }
}

// ----------------------------------------------------------------------------- attend
// grid (tokens, head groups of LA_WARPS, splits).  Warp w of a CTA owns head hg * LA_WARPS + w; a tile of
// LA_TILE cached rows is staged in shared memory as float32 once for all the CTA's heads.  Lane j scores key
// j of the tile; for the weighted sum lane l owns latent elements l, l + 32, ...
template <typename TC>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attend_kernel(const float* __restrict__ qcat, const TC* __restrict__ cache, const int* __restrict__ block_table,
                     int max_blocks, const int* __restrict__ token_req, const int* __restrict__ positions, int H, int r,
                     int dr, int page_size, float scale, int window, int splits, float* __restrict__ o_lat,
                     float* __restrict__ part_o, float* __restrict__ part_ml) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int W = r + dr, Wp = W + 1;
  float* rows = sm;                              // [LA_TILE][Wp]
  float* qsm = sm + LA_TILE * Wp;                // [LA_WARPS][W]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, h = blockIdx.y * LA_WARPS + warp, split = blockIdx.z;
  const bool live = h < H;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  const int key_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // this split's share of the key tiles
  const int tile_lo = key_lo / LA_TILE, tile_hi = pos / LA_TILE + 1;
  const int n_tiles = tile_hi - tile_lo;
  const int my_lo = tile_lo + (int)((long long)n_tiles * split / splits);
  const int my_hi = tile_lo + (int)((long long)n_tiles * (split + 1) / splits);
  float* qw = qsm + (size_t)warp * W;
  if (live) {
    const float* qg = qcat + ((size_t)t * H + h) * W;
    for (int e = lane; e < W; e += 32) qw[e] = qg[e];
  }
  float m = -INFINITY, l = 0.f;
  float o[LA_MAX_R / 32];
#pragma unroll
  for (int i = 0; i < LA_MAX_R / 32; i++) o[i] = 0.f;

  for (int tile = my_lo; tile < my_hi; tile++) {
    const int base = tile * LA_TILE;
    __syncthreads();                             // the tile before has been read by every warp
    for (int j = warp; j < LA_TILE; j += LA_WARPS) {
      int key = base + j;
      if (key < key_lo || key > pos) continue;
      const TC* src = cache + ((size_t)bt[key / page_size] * page_size + key % page_size) * W;
      for (int e = lane; e < W; e += 32) rows[j * Wp + e] = to_float(src[e]);
    }
    __syncthreads();
    if (!live) continue;
    const int key = base + lane;
    const bool valid = key >= key_lo && key <= pos;
    float s = -INFINITY;
    if (valid) {
      const float* kr = rows + lane * Wp;
      float acc = 0.f;
      for (int e = 0; e < W; e++) acc = fmaf(qw[e], kr[e], acc);
      s = acc * scale;
    }
    float m_new = fmaxf(m, warp_max(s));
    float c = expf(m - m_new);                   // m = -inf before the first key gives 0
    float p = valid ? expf(s - m_new) : 0.f;
    l = l * c + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < LA_MAX_R / 32; i++) o[i] *= c;
    const int j0 = key_lo > base ? key_lo - base : 0;
    const int j1 = pos - base + 1 < LA_TILE ? pos - base + 1 : LA_TILE;
    for (int j = j0; j < j1; j++) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vr = rows + j * Wp;
#pragma unroll
      for (int i = 0; i < LA_MAX_R / 32; i++) {
        int e = lane + 32 * i;
        if (e < r) o[i] = fmaf(pj, vr[e], o[i]);
      }
    }
  }
  if (!live) return;
  if (splits == 1) {
    float inv = 1.0f / l;
    float* dst = o_lat + ((size_t)t * H + h) * r;
#pragma unroll
    for (int i = 0; i < LA_MAX_R / 32; i++) {
      int e = lane + 32 * i;
      if (e < r) dst[e] = o[i] * inv;
    }
  } else {
    size_t item = ((size_t)t * H + h) * splits + split;
    float* dst = part_o + item * r;
#pragma unroll
    for (int i = 0; i < LA_MAX_R / 32; i++) {
      int e = lane + 32 * i;
      if (e < r) dst[e] = o[i];
    }
    if (lane == 0) { part_ml[2 * item] = m; part_ml[2 * item + 1] = l; }
  }
}

// ----------------------------------------------------------------------------- attend on tensor cores (bfloat16)
// grid (tokens, groups of 16 heads, splits); 8 warps.  The 16 heads of a token are the rows of one m16 tile: they
// share the token's keys, so one staged tile of 64 cached rows serves all of them.  Per key tile:
//   S = Q K^T      warp w takes keys 8w .. 8w+7 (one n-tile), K-dimension the whole row (latent + rotated part);
//                  the float32 queries enter as TWO bfloat16 numbers, q = hi + lo (two products, one sum)
//   softmax        float32 on S in shared memory; the weights leave as TWO bfloat16 numbers, p = hi + lo, so that
//                  the product with the values sees them to 16 bits of mantissa, not 8
//   O += P V       V is the latent part of the same staged rows (ldmatrix.trans); warp w owns columns 8j, j = w mod 8
// The next tile's rows travel by cp.async into the other buffer meanwhile; keys outside the token's range arrive
// as zeros (a copy of zero bytes).  Needs the row and the latent to be whole 16-byte pieces (multiples of 8).
#define LM_KT 64
__device__ __forceinline__ void lm_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256)
latent_attend_mma_kernel(const float* __restrict__ qcat, const bf16* __restrict__ cache,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_req,
                         const int* __restrict__ positions, int H, int r, int dr, int page_size, float scale, int window,
                         int splits, float* __restrict__ o_lat, float* __restrict__ part_o,
                         float* __restrict__ part_ml) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char lm_raw[];
  const int W = r + dr, Wq = (W + 15) & ~15, P = Wq + 8;         // pitch of a staged row in elements
  bf16* Qs = reinterpret_cast<bf16*>(lm_raw);                    // [16][P]: the queries' leading 8 bits of mantissa
  bf16* Ql = Qs + 16 * P;                                        // [16][P]: what those left out (q = hi + lo)
  bf16* Ks = Ql + 16 * P;                                        // [2][LM_KT][P]
  float* Ss = reinterpret_cast<float*>(Ks + 2 * LM_KT * P);      // [16][68]
  bf16* Ph = reinterpret_cast<bf16*>(Ss + 16 * 68);              // [16][72]
  bf16* Pl = Ph + 16 * 72;                                       // [16][72]
  float* m_s = reinterpret_cast<float*>(Pl + 16 * 72);           // [16]
  float* l_s = m_s + 16;
  float* corr_s = l_s + 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int t = blockIdx.x, h0 = blockIdx.y * 16, split = blockIdx.z;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  const int key_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int tile_lo = key_lo / LM_KT, n_tiles = pos / LM_KT + 1 - tile_lo;
  const int my_lo = tile_lo + (int)((long long)n_tiles * split / splits);
  const int my_hi = tile_lo + (int)((long long)n_tiles * (split + 1) / splits);
  const int pieces = W >> 3;                                     // 16-byte pieces of a cached row

  // a warp copies whole rows (8 of the 64 each): the page lookup once per row, then 16-byte pieces lane by lane
  auto issue = [&](int tile, int buf) {
    bf16* dst = Ks + (size_t)buf * LM_KT * P;
    for (int row = warp; row < LM_KT; row += 8) {
      const int key = tile * LM_KT + row;
      const bool ok = key >= key_lo && key <= pos;
      const bf16* src = ok ? cache + ((size_t)bt[key / page_size] * page_size + key % page_size) * W : cache;
      const unsigned d = (unsigned)__cvta_generic_to_shared(dst + row * P);
      const unsigned n = ok ? 16u : 0u;
      for (int c = lane; c < pieces; c += 32)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d + 16u * c), "l"(ok ? src + 8 * c : src), "r"(n)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  for (int i = tid; i < 16 * Wq; i += 256) {
    int row = i / Wq, e = i - row * Wq;
    float v = (h0 + row < H && e < W) ? qcat[((size_t)t * H + h0 + row) * W + e] : 0.f;
    bf16 hi = __float2bfloat16_rn(v);
    Qs[row * P + e] = hi;
    Ql[row * P + e] = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
  if (Wq > W)
    for (int i = tid; i < 2 * LM_KT * (Wq - W); i += 256) {
      int row = i / (Wq - W), e = W + i - row * (Wq - W);
      Ks[row * P + e] = __float2bfloat16_rn(0.f);
    }
  if (tid < 16) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int q = 0; q < 4; q++) acc[i][q] = 0.f;
  const int n_ntiles = r >> 3;                                   // n-tiles of 8 latent columns; warp w owns w, w + 8, ...

  if (my_lo < my_hi) issue(my_lo, 0);
  for (int tile = my_lo; tile < my_hi; tile++) {
    const int buf = (tile - my_lo) & 1;
    if (tile + 1 < my_hi) {
      issue(tile + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const bf16* Kb = Ks + (size_t)buf * LM_KT * P;
    {   // S = Q K^T for this warp's 8 keys
      // four independent sums (hi and lo, even and odd steps): one sum would chain every MMA to the one before
      float c4[4][4];
#pragma unroll
      for (int u = 0; u < 4; u++) c4[u][0] = c4[u][1] = c4[u][2] = c4[u][3] = 0.f;
      // operands by ldmatrix: the 16 x 16 piece of the queries (hi, lo) as four 8 x 8 matrices, the 8 keys x 16 as two
      const unsigned q_hi = (unsigned)__cvta_generic_to_shared(Qs + (lane & 15) * P + (lane >> 4) * 8);
      const unsigned q_lo = (unsigned)__cvta_generic_to_shared(Ql + (lane & 15) * P + (lane >> 4) * 8);
      const unsigned k_ad = (unsigned)__cvta_generic_to_shared(Kb + (warp * 8 + (lane & 7)) * P + ((lane >> 3) & 1) * 8);
      auto step = [&](int ks, float* ch, float* cl) {
        unsigned a[4], b[4], k0, k1;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(q_hi + 2u * ks));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(q_lo + 2u * ks));
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(k0), "=r"(k1) : "r"(k_ad + 2u * ks));
        lm_mma(ch, a, k0, k1);
        lm_mma(cl, b, k0, k1);
      };
      int ks = 0;
      for (; ks + 32 <= Wq; ks += 32) {
        step(ks, c4[0], c4[1]);
        step(ks + 16, c4[2], c4[3]);
      }
      if (ks < Wq) step(ks, c4[0], c4[1]);
      float c[4];
#pragma unroll
      for (int u = 0; u < 4; u++) c[u] = (c4[0][u] + c4[2][u]) + (c4[1][u] + c4[3][u]);
      const int kcol = warp * 8 + 2 * tq, key = tile * LM_KT + kcol;
      const bool v0 = key >= key_lo && key <= pos, v1 = key + 1 >= key_lo && key + 1 <= pos;
      Ss[g * 68 + kcol] = v0 ? c[0] * scale : -INFINITY;
      Ss[g * 68 + kcol + 1] = v1 ? c[1] * scale : -INFINITY;
      Ss[(g + 8) * 68 + kcol] = v0 ? c[2] * scale : -INFINITY;
      Ss[(g + 8) * 68 + kcol + 1] = v1 ? c[3] * scale : -INFINITY;
    }
    __syncthreads();
    {   // softmax of row tid / 16 over its 64 scores, 4 a thread
      const int row = tid >> 4, c0 = (tid & 15) * 4;
      float sv[4];
#pragma unroll
      for (int j = 0; j < 4; j++) sv[j] = Ss[row * 68 + c0 + j];
      float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = m_s[row], m_new = fmaxf(m_old, mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float pj = sv[j] > -INFINITY ? expf(sv[j] - m_new) : 0.f;
        sum += pj;
        bf16 hi = __float2bfloat16_rn(pj);
        Ph[row * 72 + c0 + j] = hi;
        Pl[row * 72 + c0 + j] = __float2bfloat16_rn(pj - __bfloat162float(hi));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __syncwarp();
      if ((tid & 15) == 0) {
        float corr = m_old > -INFINITY ? expf(m_old - m_new) : 0.f;
        corr_s[row] = corr;
        l_s[row] = l_s[row] * corr + sum;
        m_s[row] = m_new;
      }
    }
    __syncthreads();
    {   // O += P V
      const float cg = corr_s[g], cg8 = corr_s[g + 8];
#pragma unroll
      for (int i = 0; i < 8; i++) { acc[i][0] *= cg; acc[i][1] *= cg; acc[i][2] *= cg8; acc[i][3] *= cg8; }
#pragma unroll
      for (int kk = 0; kk < LM_KT; kk += 16) {
        unsigned ah[4], al[4];
        const unsigned p_hi = (unsigned)__cvta_generic_to_shared(Ph + (lane & 15) * 72 + kk + (lane >> 4) * 8);
        const unsigned p_lo = (unsigned)__cvta_generic_to_shared(Pl + (lane & 15) * 72 + kk + (lane >> 4) * 8);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(ah[0]), "=r"(ah[1]), "=r"(ah[2]), "=r"(ah[3]) : "r"(p_hi));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(al[0]), "=r"(al[1]), "=r"(al[2]), "=r"(al[3]) : "r"(p_lo));
        const bf16* vrow = Kb + (size_t)(kk + (lane & 15)) * P;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int j = warp + 8 * i;
          if (j < n_ntiles) {
            unsigned b0, b1;
            unsigned addr = (unsigned)__cvta_generic_to_shared(vrow + j * 8);
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(addr));
            lm_mma(acc[i], ah, b0, b1);
            lm_mma(acc[i], al, b0, b1);
          }
        }
      }
    }
    __syncthreads();                                             // the buffer may be filled again
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int j = warp + 8 * i;
    if (j >= n_ntiles) continue;
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int row = g + (q >> 1) * 8, h = h0 + row, col = j * 8 + 2 * tq + (q & 1);
      if (h >= H) continue;
      if (splits == 1) o_lat[((size_t)t * H + h) * r + col] = acc[i][q] / l_s[row];
      else part_o[(((size_t)t * H + h) * splits + split) * r + col] = acc[i][q];
    }
  }
  if (splits > 1 && tid < 16 && h0 + tid < H) {
    size_t item = ((size_t)t * H + h0 + tid) * splits + split;
    part_ml[2 * item] = m_s[tid];
    part_ml[2 * item + 1] = l_s[tid];
  }
}

// o_lat[t, h] = sum_s exp(m_s - M) o_s / sum_s exp(m_s - M) l_s; a split without keys has m = -inf and l = 0.
__global__ void latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                      int r, float* __restrict__ o_lat) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t item = blockIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < splits; s++) M = fmaxf(M, part_ml[2 * (item * splits + s)]);
  float L = 0.f;
  for (int s = 0; s < splits; s++) {
    float ms = part_ml[2 * (item * splits + s)];
    if (ms > -INFINITY) L += expf(ms - M) * part_ml[2 * (item * splits + s) + 1];
  }
  for (int e = threadIdx.x; e < r; e += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; s++) {
      float ms = part_ml[2 * (item * splits + s)];
      if (ms > -INFINITY) acc = fmaf(expf(ms - M), part_o[(item * splits + s) * r + e], acc);
    }
    o_lat[item * r + e] = acc / L;
  }
}

// ----------------------------------------------------------------------------- expand
// out[t, h * dv + i] = (sum_j Wuv[h * dv + i, j] o_lat[t, h, j]) * sigmoid(gate[t, h * dv + i]); gate float32 with
// row stride ldg (null: no gate).  A warp per output row of Wuv, LA_TT tokens and 32 output rows a CTA.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
latent_expand_kernel(const float* __restrict__ o_lat, const TW* __restrict__ wuv, const float* __restrict__ gate,
                     long long ldg, TO* __restrict__ out, int T, int H, int dv, int r, int vec,
                     const float* __restrict__ pre) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float os[];                // [LA_TT][r]
  const int h = blockIdx.y, t0 = blockIdx.x * LA_TT;
  const int nt = min(LA_TT, T - t0);
  const int i_hi = min(dv, (int)(blockIdx.z + 1) * 32);
  if (pre) {            // Wuv_h o_lat was made elsewhere ([H, T, dv]): the gate and the rounding are left
    for (int k = threadIdx.x; k < nt * 32; k += blockDim.x) {
      int tt = k >> 5, i = blockIdx.z * 32 + (k & 31);
      if (i >= i_hi) continue;
      float v = pre[((size_t)h * T + t0 + tt) * dv + i];
      if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)(t0 + tt) * ldg + (size_t)h * dv + i]));
      out[(size_t)(t0 + tt) * H * dv + (size_t)h * dv + i] = from_float<TO>(v);
    }
    return;
  }
  for (int i = threadIdx.x; i < LA_TT * r; i += blockDim.x) {
    int tt = i / r, j = i - tt * r;
    os[i] = tt < nt ? o_lat[((size_t)(t0 + tt) * H + h) * r + j] : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int i = blockIdx.z * 32 + warp; i < i_hi; i += nw) {
    const TW* wrow = wuv + ((size_t)h * dv + i) * r;
    float acc[LA_TT];
#pragma unroll
    for (int tt = 0; tt < LA_TT; tt++) acc[tt] = 0.f;
    if (vec) {
      constexpr int V = Vec16<TW>::N;
      for (int j = lane * V; j < r; j += 32 * V) {
        float w[V];
        Vec16<TW>::load(wrow + j, w);
#pragma unroll
        for (int tt = 0; tt < LA_TT; tt++)
#pragma unroll
          for (int v = 0; v < V; v++) acc[tt] = fmaf(w[v], os[tt * r + j + v], acc[tt]);
      }
    } else {
      for (int j = lane; j < r; j += 32) {
        float w = to_float(wrow[j]);
#pragma unroll
        for (int tt = 0; tt < LA_TT; tt++) acc[tt] = fmaf(w, os[tt * r + j], acc[tt]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < LA_TT; tt++) acc[tt] = warp_sum(acc[tt]);
    if (lane == 0) {
#pragma unroll
      for (int tt = 0; tt < LA_TT; tt++) {
        if (tt >= nt) continue;
        float v = acc[tt];
        if (gate) {
          float g = gate[(size_t)(t0 + tt) * ldg + (size_t)h * dv + i];
          v *= 1.0f / (1.0f + expf(-g));
        }
        out[(size_t)(t0 + tt) * H * dv + (size_t)h * dv + i] = from_float<TO>(v);
      }
    }
  }
}

// ----------------------------------------------------------------------------- launchers
// QD_LATENT_MMA=0 in the environment keeps the float32-FMA attend kernel in bfloat16 too (to compare the two).
static inline bool lm_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("QD_LATENT_MMA");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

extern "C" int qd_latent_prep(const float* u, long long ldu, int q_off, int q_rank, int kv_off, int r, int dr,
                              const float* wq_norm, const float* wkv_norm, float eps, const float* cos_t,
                              const float* sin_t, int rot_dims, const int* positions, const int* slot_map, void* cq,
                              void* cache, int dtype, int write_cache, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot_dims % 2 || rot_dims > dr || q_rank < 0 || r <= 0) return QD_ERR_UNSUPPORTED;
  if (dtype == QD_F32)
    qd_launch(latent_prep_kernel<float>, dim3(T), dim3(256), 0, stream, u, ldu, q_off, q_rank, kv_off, r, dr, wq_norm,
              wkv_norm, eps, cos_t, sin_t, rot_dims, positions, slot_map, (float*)cq, (float*)cache, write_cache);
  else if (dtype == QD_BF16)
    qd_launch(latent_prep_kernel<bf16>, dim3(T), dim3(256), 0, stream, u, ldu, q_off, q_rank, kv_off, r, dr, wq_norm,
              wkv_norm, eps, cos_t, sin_t, rot_dims, positions, slot_map, (bf16*)cq, (bf16*)cache, write_cache);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// ``pre`` (float32 [H, T, r], or null): Wuk_h^T q_h already made by a batched library product; the kernel then only
// lays it beside the rotated part.
extern "C" int qd_latent_absorb(const float* q, long long ldq, const void* wuk, int w_dtype, float* qcat, int T, int H, int dn, int dr,
                                int r, const float* cos_t, const float* sin_t, int rot_dims, const int* positions,
                                const float* pre, cudaStream_t stream) {
  if (T <= 0) return 0;
  size_t smem = (size_t)LA_TT * dn * sizeof(float);
  if (smem > 48 * 1024 || H > 65535) return QD_ERR_UNSUPPORTED;
  {
    const int V = w_dtype == QD_F32 ? 4 : 8;
    const size_t vsm = (size_t)LA_TT * (dn + r) * sizeof(float);
    if (!pre && (w_dtype == QD_F32 || w_dtype == QD_BF16) && r % V == 0 && r / V <= 256 && 256 % (r / V) == 0 &&
        !((uintptr_t)wuk & 15) && vsm <= 48 * 1024) {
      dim3 vgrid((T + LA_TT - 1) / LA_TT, H);
      if (w_dtype == QD_F32)
        qd_launch(latent_absorb_vec_kernel<float>, vgrid, dim3(256), vsm, stream, q, ldq, (const float*)wuk, qcat, T, H, dn, dr,
                  r, cos_t, sin_t, rot_dims, positions);
      else
        qd_launch(latent_absorb_vec_kernel<bf16>, vgrid, dim3(256), vsm, stream, q, ldq, (const bf16*)wuk, qcat, T, H, dn, dr,
                  r, cos_t, sin_t, rot_dims, positions);
      return qd_last_error();
    }
  }
  dim3 grid((T + LA_TT - 1) / LA_TT, H, (r + 255) / 256);
  if (w_dtype == QD_F32)
    qd_launch(latent_absorb_kernel<float>, grid, dim3(256), smem, stream, q, ldq, (const float*)wuk, qcat, T, H, dn, dr, r,
              cos_t, sin_t, rot_dims, positions, pre);
  else if (w_dtype == QD_BF16)
    qd_launch(latent_absorb_kernel<bf16>, grid, dim3(256), smem, stream, q, ldq, (const bf16*)wuk, qcat, T, H, dn, dr, r,
              cos_t, sin_t, rot_dims, positions, pre);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

extern "C" int qd_latent_attend(const float* qcat, const void* cache, int dtype, const int* block_table, int max_blocks,
                                const int* token_req, const int* positions, int T, int H, int r, int dr, int page_size,
                                float scale, int window, int splits, float* o_lat, float* part_o, float* part_ml,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (r > LA_MAX_R || r <= 0 || splits < 1 || splits > 65535 || H > 65535 * LA_WARPS || page_size <= 0) return QD_ERR_UNSUPPORTED;
  if (splits > 1 && (!part_o || !part_ml)) return QD_ERR_UNSUPPORTED;
  const int W = r + dr;
  if (dtype == QD_BF16 && lm_enabled() && W % 8 == 0 && r % 8 == 0 && !((uintptr_t)cache & 15)) {
    const int P = ((W + 15) & ~15) + 8;
    size_t sm = (size_t)(32 + 2 * LM_KT) * P * 2 + 16 * 68 * 4 + 2 * 16 * 72 * 2 + 48 * 4;
    if (sm <= 220 * 1024 && H <= 65535 * 16) {
      static bool attr_set = false;
      if (!attr_set) {
        cudaFuncSetAttribute(latent_attend_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        attr_set = true;
      }
      qd_launch(latent_attend_mma_kernel, dim3(T, (H + 15) / 16, splits), dim3(256), sm, stream, qcat, (const bf16*)cache,
                block_table, max_blocks, token_req, positions, H, r, dr, page_size, scale, window, splits, o_lat, part_o,
                part_ml);
      if (splits > 1)
        qd_launch(latent_combine_kernel, dim3((unsigned)((size_t)T * H)), dim3(128), 0, stream, (const float*)part_o,
                  (const float*)part_ml, splits, r, o_lat);
      return qd_last_error();
    }
  }
  size_t smem = ((size_t)LA_TILE * (W + 1) + (size_t)LA_WARPS * W) * sizeof(float);
  if (smem > 200 * 1024) return QD_ERR_UNSUPPORTED;
  dim3 grid(T, (H + LA_WARPS - 1) / LA_WARPS, splits);
#define LA_GO(TC)                                                                                                  \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(latent_attend_kernel<TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    qd_launch(latent_attend_kernel<TC>, grid, dim3(LA_WARPS * 32), smem, stream, qcat, (const TC*)cache, block_table, \
              max_blocks, token_req, positions, H, r, dr, page_size, scale, window, splits, o_lat, part_o, part_ml); \
  } while (0)
  if (dtype == QD_F32) LA_GO(float);
  else if (dtype == QD_BF16) LA_GO(bf16);
  else return QD_ERR_UNSUPPORTED;
#undef LA_GO
  if (splits > 1)
    qd_launch(latent_combine_kernel, dim3((unsigned)((size_t)T * H)), dim3(128), 0, stream, (const float*)part_o,
              (const float*)part_ml, splits, r, o_lat);
  return qd_last_error();
}

extern "C" int qd_latent_expand(const float* o_lat, const void* wuv, int w_dtype, const float* gate, long long ldg,
                                void* out, int out_dtype, int T, int H, int dv, int r, const float* pre,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  size_t smem = (size_t)LA_TT * r * sizeof(float);
  if (smem > 48 * 1024 || H > 65535) return QD_ERR_UNSUPPORTED;
  dim3 grid((T + LA_TT - 1) / LA_TT, H, (dv + 31) / 32);
  const int vec = (r % (w_dtype == QD_F32 ? 4 : 8) == 0 && !((uintptr_t)wuv & 15)) ? 1 : 0;     // rows in 16-byte pieces
  if (w_dtype == QD_F32 && out_dtype == QD_F32)
    qd_launch(latent_expand_kernel<float, float>, grid, dim3(256), smem, stream, o_lat, (const float*)wuv, gate, ldg,
              (float*)out, T, H, dv, r, vec, pre);
  else if (w_dtype == QD_BF16 && out_dtype == QD_BF16)
    qd_launch(latent_expand_kernel<bf16, bf16>, grid, dim3(256), smem, stream, o_lat, (const bf16*)wuv, gate, ldg,
              (bf16*)out, T, H, dv, r, vec, pre);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// ---------------------------------------------------------------------------------- rows for the expanded form
// For prompt portions the keys and values of all heads are expanded from the cached rows by one product, and an
// ordinary attention kernel runs over them.  ``latent_gather`` lays the first r elements of every cached row of the
// requests' contexts out densely, request by request with Lmax rows each (rows past a request's context are zero):
//   out[(q * Lmax + j), :] = cache row j of request q,  j < start_pos[q] + tokens of q in this step
// grid (Lmax, requests), 128 threads.
template <typename T>
__global__ void __launch_bounds__(128)
latent_gather_kernel(const T* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
                     const int* __restrict__ cu_tokens, const int* __restrict__ start_pos, int page_size, int W, int r,
                     T* __restrict__ out, int Lmax) {
  pdl_launch_dependents();
  pdl_wait();
  const int j = blockIdx.x, q = blockIdx.y;
  const int len = start_pos[q] + cu_tokens[q + 1] - cu_tokens[q];
  T* o = out + ((size_t)q * Lmax + j) * r;
  if (j >= len) {
    for (int i = threadIdx.x; i < r; i += blockDim.x) o[i] = from_float<T>(0.f);
    return;
  }
  const int page = block_table[(size_t)q * max_blocks + j / page_size];
  const T* src = cache + ((size_t)page * page_size + j % page_size) * W;
  for (int i = threadIdx.x; i < r; i += blockDim.x) o[i] = src[i];
}

extern "C" int qd_latent_gather(const void* cache, int dtype, const int* block_table, int max_blocks,
                                const int* cu_tokens, const int* start_pos, int n_requests, int page_size, int W, int r,
                                void* out, int Lmax, cudaStream_t stream) {
  if (n_requests <= 0 || Lmax <= 0) return 0;
  if (n_requests > 65535 || r <= 0 || r > W || page_size <= 0) return QD_ERR_UNSUPPORTED;
  dim3 grid(Lmax, n_requests);
  if (dtype == QD_BF16)
    qd_launch(latent_gather_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)cache, block_table, max_blocks,
              cu_tokens, start_pos, page_size, W, r, (bf16*)out, Lmax);
  else if (dtype == QD_F32)
    qd_launch(latent_gather_kernel<float>, grid, dim3(128), 0, stream, (const float*)cache, block_table, max_blocks,
              cu_tokens, start_pos, page_size, W, r, (float*)out, Lmax);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// out[t, 0..N) = in[t, 0..N) rounded to bfloat16 (in float32, rows ldin apart; out dense).
__global__ void __launch_bounds__(256)
round_rows_kernel(const float* __restrict__ in, long long ldin, bf16* __restrict__ out, int N, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / N;
  out[i] = __float2bfloat16_rn(in[t * ldin + (i - t * N)]);
}

extern "C" int qd_round_rows(const float* in, long long ldin, void* out, int T, int N, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  const size_t n = (size_t)T * N;
  qd_launch(round_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, in, ldin, (bf16*)out, N, n);
  return qd_last_error();
}
