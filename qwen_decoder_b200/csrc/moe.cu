// A feed-forward of routed experts.
//
//   route    logits = Wr h + b in float32 (one warp per token); the ``top`` largest (the lower index wins a tie);
//            weights = softmax over the chosen logits; also sigmoid(Wsg h), the gate of a shared expert
//   sort     the (token, choice) pairs ordered by expert: for each expert the range of its pairs, for each pair its
//            place, and a table of row tiles (expert, first row, rows) for the grouped products
//   gate_up  act[place] = silu(Wg_e x) * (Wu_e x) for every pair, x = the pair's token        } grouped products:
//   down     y[place] = Wd_e act[place]                                    float32            } a tile = one expert
//   combine  out[t] = sum_k weight[t, k] y[place(t, k)] + gate[t] * shared[t]                  float32
//
// Variants, all parameters of the launchers: the router may instead take the softmax over ALL its outputs, choose by
// score + a per-output correction and weigh by the plain score (``route_mode`` 1); the last outputs of the router
// may be identity experts, which have no weights and whose output is the token's input itself (they get no row
// tiles; combine adds weight * input); the gated activation may be the clamped form
// min(g, L) * sigmoid(a * min(g, L)) * (clamp(u, -L, L) + 1) (``act`` 1) instead of silu(g) * u.  ``route_mode`` 2 chooses
// the ``top`` largest logits and weighs each by its own sigmoid, not renormalised.  A pair's weight may multiply the
// expert's INPUT instead of its output (``in_scale`` of the gated product: W (w h) = w (W h), so both sums of the pair
// are multiplied by w before the gate; combine then adds the pairs' outputs as they are).
//
// Nothing comes back to the host between these: counts, places and tiles stay on the device, so a step with
// routed experts is captured in a CUDA graph like any other.  The products run on float32 FMA with the
// weights in the engine's dtype; a tile's rows are pairs of one expert, its sums one FMA chain over k each.
#include "common.cuh"

#define MOE_MAX_TOP 32

// The gate of a gated expert: act 0 silu(g) * u; act 1 the clamped form with slope ``alpha`` and limit ``limit``.
struct MoeAct { int kind; float limit, alpha; };
__device__ __forceinline__ float moe_gated(float g, float u, MoeAct a) {
  if (a.kind == 0) return g / (1.0f + expf(-g)) * u;
  g = fminf(g, a.limit);
  u = fminf(fmaxf(u, -a.limit), a.limit);
  return g / (1.0f + expf(-a.alpha * g)) * (u + 1.0f);
}

// ----------------------------------------------------------------------------- route
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

#define MR_TOKENS 8
// logits[t, e] = wr[e] . h[t] + br[e] in float32; row E of the output (when wsg is given) is sigmoid(wsg . h[t]).
// grid (token tiles of MR_TOKENS, groups of 8 rows of wr): a warp owns one row of wr and reads it once for the tile.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
moe_logits_kernel(const T* __restrict__ h, const T* __restrict__ wr, const float* __restrict__ br,
                  const T* __restrict__ wsg, int n_tokens, int D, int E, float* __restrict__ logits,
                  float* __restrict__ sgate) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.y * 8 + warp, t0 = blockIdx.x * MR_TOKENS;
  const int rows = E + (wsg ? 1 : 0);
  if (e >= rows) return;
  const T* w = e < E ? wr + (size_t)e * D : wsg;
  const int nt = min(MR_TOKENS, n_tokens - t0);
  float acc[MR_TOKENS];
#pragma unroll
  for (int i = 0; i < MR_TOKENS; i++) acc[i] = 0.f;
  if (VEC) {
    constexpr int V = Vec16<T>::N;
    for (int k = lane * V; k < D; k += 32 * V) {
      float wv[V], xv[V];
      Vec16<T>::load(w + k, wv);
#pragma unroll
      for (int i = 0; i < MR_TOKENS; i++) {
        if (i < nt) {
          Vec16<T>::load(h + (size_t)(t0 + i) * D + k, xv);
#pragma unroll
          for (int j = 0; j < V; j++) acc[i] = fmaf(xv[j], wv[j], acc[i]);
        }
      }
    }
  } else {
    for (int k = lane; k < D; k += 32) {
      float wv = to_float(w[k]);
#pragma unroll
      for (int i = 0; i < MR_TOKENS; i++)
        if (i < nt) acc[i] = fmaf(to_float(h[(size_t)(t0 + i) * D + k]), wv, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < MR_TOKENS; i++) {
    float v = warp_sum(acc[i]);
    if (lane == 0 && i < nt) {
      if (e < E) logits[(size_t)(t0 + i) * E + e] = v + (br ? br[e] : 0.0f);
      else sgate[t0 + i] = 1.0f / (1.0f + expf(-v));
    }
  }
}

// One thread per token.  mode 0: the ``top`` largest logits (the lower index wins a tie) and the softmax over them.
// mode 1: scores = softmax over all E logits; the ``top`` largest of score + corr[e] are chosen (the lower index wins
// a tie); the weights are the chosen outputs' plain scores, not renormalised.  mode 2: the ``top`` largest logits, each
// weighed by sigmoid(logit).
__global__ void __launch_bounds__(128)
moe_topk_kernel(float* __restrict__ logits, int n_tokens, int E, int top, int mode, const float* __restrict__ corr,
                int* __restrict__ idx, float* __restrict__ wt) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  float* my = logits + (size_t)t * E;
  float v[MOE_MAX_TOP];
  if (mode == 1) {
    float zmax = -INFINITY, sum = 0.f;
    for (int e = 0; e < E; e++) zmax = fmaxf(zmax, my[e]);
    for (int e = 0; e < E; e++) sum += expf(my[e] - zmax);
    const float inv = 1.0f / sum;
    for (int e = 0; e < E; e++) my[e] = expf(my[e] - zmax) * inv;        // the scores, in place
    for (int k = 0; k < top; k++) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; e++) {
        float s = my[e];
        if (s < 0.f) continue;                                           // taken already
        float c = s + (corr ? corr[e] : 0.f);
        if (best < 0 || c > bv) { best = e; bv = c; }
      }
      idx[(size_t)t * top + k] = best;
      wt[(size_t)t * top + k] = my[best];
      my[best] = -1.0f;
    }
    return;
  }
  for (int k = 0; k < top; k++) {
    int best = -1;
    float bv = -INFINITY;
    for (int e = 0; e < E; e++) {
      float z = my[e];
      if (best < 0 || z > bv) { best = e; bv = z; }
    }
    idx[(size_t)t * top + k] = best;
    v[k] = bv;
    my[best] = -INFINITY;
  }
  if (mode == 2) {                                // each chosen output's own sigmoid
    for (int k = 0; k < top; k++) wt[(size_t)t * top + k] = 1.0f / (1.0f + expf(-v[k]));
    return;
  }
  float sum = 0.f;
  const float vmax = v[0];                        // the first chosen is the largest
  for (int k = 0; k < top; k++) { v[k] = expf(v[k] - vmax); sum += v[k]; }
  for (int k = 0; k < top; k++) wt[(size_t)t * top + k] = v[k] / sum;
}

// The same choice with one warp per token (up to 256 router outputs: eight per lane, in registers): the softmax's
// maximum and sum and every round's best output are warp reductions.  A round picks the largest value; of equal
// values the lower index.
#define MT_PER_LANE 8
__global__ void __launch_bounds__(128)
moe_topk_warp_kernel(const float* __restrict__ logits, int n_tokens, int E, int top, int mode,
                     const float* __restrict__ corr, int* __restrict__ idx, float* __restrict__ wt) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  const float* my = logits + (size_t)t * E;
  float z[MT_PER_LANE], c[MT_PER_LANE];         // the value a weight is made from, and the value the choice goes by
  float zmax = -INFINITY;
#pragma unroll
  for (int j = 0; j < MT_PER_LANE; j++) {
    const int e = lane + 32 * j;
    z[j] = e < E ? my[e] : -INFINITY;
    zmax = fmaxf(zmax, z[j]);
  }
  zmax = warp_max(zmax);
  if (mode == 1) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MT_PER_LANE; j++) { z[j] = lane + 32 * j < E ? expf(z[j] - zmax) : 0.f; sum += z[j]; }
    const float inv = 1.0f / warp_sum(sum);
#pragma unroll
    for (int j = 0; j < MT_PER_LANE; j++) {
      const int e = lane + 32 * j;
      z[j] *= inv;                              // the score
      c[j] = e < E ? z[j] + (corr ? corr[e] : 0.f) : -INFINITY;
    }
  } else {
#pragma unroll
    for (int j = 0; j < MT_PER_LANE; j++) c[j] = z[j];
  }
  float chosen = 0.f, first = 0.f, sum = 0.f;   // lane k keeps what round k chose
  for (int k = 0; k < top; k++) {
    float bv = -INFINITY, bz = 0.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MT_PER_LANE; j++)       // ascending index within a lane: '>' keeps the lower one
      if (c[j] > bv) { bv = c[j]; be = lane + 32 * j; bz = z[j]; }
    if (bv == -INFINITY) be = 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o), oz = __shfl_xor_sync(0xffffffffu, bz, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; bz = oz; }
    }
#pragma unroll
    for (int j = 0; j < MT_PER_LANE; j++)
      if (lane + 32 * j == be) c[j] = -INFINITY;
    if (k == 0) first = bz;
    // mode 0: the first chosen is the largest logit; mode 2: the chosen logit's own sigmoid
    const float w = mode == 1 ? bz : mode == 2 ? 1.0f / (1.0f + expf(-bz)) : expf(bz - first);
    sum += w;
    if (lane == (k & 31)) {
      idx[(size_t)t * top + k] = be;
      if (mode != 0) wt[(size_t)t * top + k] = w;
      else chosen = w;                          // top <= 32: one round per lane
    }
  }
  if (mode == 0 && lane < top) wt[(size_t)t * top + lane] = chosen / sum;
}

// ----------------------------------------------------------------------------- sort
// One CTA.  meta: [0, E] offsets (E + 1), then n_tiles, then tiles (expert, first row, rows) x max_tiles.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int E, int E_real, int tile_rows, int max_tiles,
                int* __restrict__ place, int* __restrict__ pair_at, int* __restrict__ meta) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int cnt[];                  // [E] counts, then [E] cursors
  int* cur = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    int* tiles = meta + E + 2;
    for (int e = 0; e < E; e++) {
      meta[e] = off;
      cur[e] = off;
      for (int r0 = 0; e < E_real && r0 < cnt[e] && nt < max_tiles; r0 += tile_rows) {   // identity experts: no tiles
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = off + r0;
        tiles[3 * nt + 2] = min(tile_rows, cnt[e] - r0);
        nt++;
      }
      off += cnt[e];
    }
    meta[E] = off;
    meta[E + 1] = nt;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    int at = atomicAdd(&cur[idx[p]], 1);
    place[p] = at;
    pair_at[at] = p;
  }
}

// ----------------------------------------------------------------------------- grouped products
// Tile of TM rows x 64 columns; 256 threads, each (TM / 16) x 4 outputs.  GATED: two weight matrices and the
// SwiGLU of their sums.  Rows of A: the pair's token (``pair_at[row] / top``) when ``by_token``, else the row itself.
template <typename TI, typename TW, typename TO, int TM, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TI* __restrict__ A, long long lda, const int* __restrict__ pair_at, int top, int by_token,
                const TW* __restrict__ W1, const TW* __restrict__ W2, TO* __restrict__ out, int N, int K,
                const int* __restrict__ meta, int E, MoeAct act, const float* __restrict__ in_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_tiles = meta[E + 1];
  if ((int)blockIdx.y >= n_tiles) return;
  const int* tile = meta + E + 2 + 3 * blockIdx.y;
  const int e = tile[0], row0 = tile[1], rows = tile[2];
  constexpr int RPT = TM / 16;                  // rows per thread
  __shared__ float As[16][TM + 4];
  __shared__ float B1[16][64 + 4];
  __shared__ float B2[GATED ? 16 : 1][64 + 4];
  __shared__ int src[TM];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int n0 = blockIdx.x * 64;
  if (tid < TM) {
    int r = row0 + tid;
    src[tid] = tid < rows ? (by_token ? pair_at[r] / top : r) : -1;
  }
  __syncthreads();
  const TW* w1 = W1 + (size_t)e * N * K;
  const TW* w2 = GATED ? W2 + (size_t)e * N * K : nullptr;
  float acc1[RPT][4], acc2[RPT][4];
#pragma unroll
  for (int i = 0; i < RPT; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc1[i][j] = acc2[i][j] = 0.f;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gk = k0 + lk + j, gn = n0 + lr;
      if (lr < TM) As[lk + j][lr] = (src[lr] >= 0 && gk < K) ? to_float(A[(size_t)src[lr] * lda + gk]) : 0.f;
      B1[lk + j][lr] = (gn < N && gk < K) ? to_float(w1[(size_t)gn * K + gk]) : 0.f;
      if (GATED) B2[lk + j][lr] = (gn < N && gk < K) ? to_float(w2[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; kk++) {
      float a[RPT], b1[4], b2[4];
#pragma unroll
      for (int i = 0; i < RPT; i++) a[i] = As[kk][ty * RPT + i];
#pragma unroll
      for (int j = 0; j < 4; j++) { b1[j] = B1[kk][tx * 4 + j]; b2[j] = GATED ? B2[kk][tx * 4 + j] : 0.f; }
#pragma unroll
      for (int i = 0; i < RPT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
          acc1[i][j] = fmaf(a[i], b1[j], acc1[i][j]);
          if (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    int r = ty * RPT + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      const float sc = in_scale ? in_scale[pair_at[row0 + r]] : 1.0f;
      float v = acc1[i][j] * sc;
      if (GATED) v = moe_gated(v, acc2[i][j] * sc, act);
      out[(size_t)(row0 + r) * N + gn] = from_float<TO>(v);
    }
  }
}

// ----------------------------------------------------------------------------- few rows per expert
// While an expert sees at most MG_ROWS pairs of a step (decoding), its weights are what the step reads: a warp
// owns output rows of the expert's matrix, reads each once in 16-byte pieces, and multiplies it with the tile's
// rows, which lie in shared memory.  grid (ceil(N / 64), tiles).
#define MG_ROWS 8
template <typename TI, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemv_kernel(const TI* __restrict__ A, long long lda, const int* __restrict__ pair_at, int top, int by_token,
                const TW* __restrict__ W1, const TW* __restrict__ W2, TO* __restrict__ out, int N, int K,
                const int* __restrict__ meta, int E, MoeAct act, const float* __restrict__ in_scale) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.y >= meta[E + 1]) return;
  const int* tile = meta + E + 2 + 3 * blockIdx.y;
  const int e = tile[0], row0 = tile[1], rows = tile[2];
  extern __shared__ __align__(16) unsigned char mg_raw[];
  TI* xs = reinterpret_cast<TI*>(mg_raw);        // [MG_ROWS][K]
  constexpr int VI = Vec16<TI>::N;
  for (int i = threadIdx.x * VI; i < rows * K; i += blockDim.x * VI) {
    int r = i / K, k = i - r * K;
    int src = by_token ? pair_at[row0 + r] / top : row0 + r;
    *reinterpret_cast<uint4*>(xs + (size_t)r * K + k) = *reinterpret_cast<const uint4*>(A + (size_t)src * lda + k);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int V = Vec16<TW>::N;                // TI and TW are the same type in every instantiation
  // two output rows at a time: twice the loads in flight for the same registers of x
  for (int i = 0; i < 8; i += 2) {
    const int n = blockIdx.x * 64 + warp * 8 + i;
    if (n >= N) break;
    const bool two = n + 1 < N;
    const TW* w1a = W1 + ((size_t)e * N + n) * K;
    const TW* w1b = two ? w1a + K : w1a;
    const TW* w2a = GATED ? W2 + ((size_t)e * N + n) * K : nullptr;
    const TW* w2b = GATED ? (two ? w2a + K : w2a) : nullptr;
    float a1[2][MG_ROWS], a2[2][MG_ROWS];
#pragma unroll
    for (int r = 0; r < MG_ROWS; r++) a1[0][r] = a1[1][r] = a2[0][r] = a2[1][r] = 0.f;
    for (int k = lane * V; k < K; k += 32 * V) {
      float wa[V], wb[V], ga[V], gb[V], xv[V];
      Vec16<TW>::load(w1a + k, wa);
      Vec16<TW>::load(w1b + k, wb);
      if (GATED) { Vec16<TW>::load(w2a + k, ga); Vec16<TW>::load(w2b + k, gb); }
#pragma unroll
      for (int r = 0; r < MG_ROWS; r++) {
        if (r < rows) {
          Vec16<TI>::load(xs + (size_t)r * K + k, xv);
#pragma unroll
          for (int j = 0; j < V; j++) {
            a1[0][r] = fmaf(xv[j], wa[j], a1[0][r]);
            a1[1][r] = fmaf(xv[j], wb[j], a1[1][r]);
            if (GATED) { a2[0][r] = fmaf(xv[j], ga[j], a2[0][r]); a2[1][r] = fmaf(xv[j], gb[j], a2[1][r]); }
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {
      if (u == 1 && !two) break;
#pragma unroll
      for (int r = 0; r < MG_ROWS; r++) {
        if (r < rows) {
          const float sc = in_scale ? in_scale[pair_at[row0 + r]] : 1.0f;
          float v = warp_sum(a1[u][r]) * sc;
          if (GATED) v = moe_gated(v, warp_sum(a2[u][r]) * sc, act);
          if (lane == 0) out[(size_t)(row0 + r) * N + n + u] = from_float<TO>(v);
        }
      }
    }
  }
}

// ----------------------------------------------------------------------------- many rows per expert, bfloat16
// Tiles of 64 pairs x 64 output columns on the tensor cores (mma.sync m16n8k16, bfloat16 in, float32 sums), K in
// steps of 64 through two stages of shared memory, the next step's 16-byte pieces on their way (cp.async) while this
// one multiplies.  Four warps, each 16 rows x 64 columns.  K must be a multiple of 8.
__device__ __forceinline__ void mma_bf16_16816(float* c, const unsigned* a, const unsigned* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void mm_ldmatrix_x4(unsigned* r, const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

__device__ __forceinline__ void mm_cp_async16(void* smem, const void* gmem, int src_bytes) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}

#define MM_KS 64            // elements of K per step through shared memory
#define MM_LD (MM_KS + 8)    // row pitch of a step in shared memory (bfloat16): no bank conflicts
#define MM_PER (MM_KS / 16)  // 16-byte pieces of each tile a thread moves per step: 64 rows x MM_KS / 8 pieces over 128 threads
template <typename TO, bool GATED>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16* __restrict__ A, long long lda, const int* __restrict__ pair_at, int top, int by_token,
                    const bf16* __restrict__ W1, const bf16* __restrict__ W2, TO* __restrict__ out, int N, int K,
                    const int* __restrict__ meta, int E, MoeAct act, const float* __restrict__ in_scale) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.y >= meta[E + 1]) return;
  const int* tile = meta + E + 2 + 3 * blockIdx.y;
  const int e = tile[0], row0 = tile[1], rows = tile[2];
  // two stages of (A rows, W1 columns[, W2 columns]), each [64][MM_LD], filled by 16-byte cp.async
  extern __shared__ __align__(16) unsigned char mm_raw[];
  constexpr int TILE = 64 * MM_LD;
  bf16* As_ = reinterpret_cast<bf16*>(mm_raw);
  bf16* B1_ = As_ + 2 * TILE;
  bf16* B2_ = B1_ + 2 * TILE;
  __shared__ int src[64];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int n0 = blockIdx.x * 64;
  if (tid < 64) src[tid] = tid < rows ? (by_token ? pair_at[row0 + tid] / top : row0 + tid) : -1;
  __syncthreads();
  const bf16* w1 = W1 + (size_t)e * N * K;
  const bf16* w2 = GATED ? W2 + (size_t)e * N * K : nullptr;
  // each thread moves MM_PER 16-byte pieces of each tile per step: piece p = tid + 128 * i -> row p / (MM_KS / 8),
  // k (p % (MM_KS / 8)) * 8; a piece outside the tile's rows, the matrix's columns or K is filled with zeros
  auto fetch = [&](int k0, int st) {
#pragma unroll
    for (int i = 0; i < MM_PER; i++) {
      const int p = tid + 128 * i, row = p / (MM_KS / 8), kc = (p % (MM_KS / 8)) * 8, k = k0 + kc;
      const bool oka = src[row] >= 0 && k < K, okb = n0 + row < N && k < K;
      mm_cp_async16(As_ + st * TILE + row * MM_LD + kc, oka ? A + (size_t)src[row] * lda + k : A, oka ? 16 : 0);
      mm_cp_async16(B1_ + st * TILE + row * MM_LD + kc, okb ? w1 + (size_t)(n0 + row) * K + k : w1, okb ? 16 : 0);
      if (GATED) mm_cp_async16(B2_ + st * TILE + row * MM_LD + kc, okb ? w2 + (size_t)(n0 + row) * K + k : w2, okb ? 16 : 0);
    }
  };
  float c1[8][4], c2[GATED ? 8 : 1][4];
#pragma unroll
  for (int j = 0; j < 8; j++)
#pragma unroll
    for (int q = 0; q < 4; q++) { c1[j][q] = 0.f; if (GATED) c2[j][q] = 0.f; }
  fetch(0, 0);
  asm volatile("cp.async.commit_group;\n" ::);
  for (int k0 = 0, st = 0; k0 < K; k0 += MM_KS, st ^= 1) {
    if (k0 + MM_KS < K) fetch(k0 + MM_KS, st ^ 1);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);  // this step's pieces have arrived (the next step's may be in flight)
    __syncthreads();
    const bf16* As = As_ + st * TILE;
    const bf16* B1 = B1_ + st * TILE;
    const bf16* B2 = B2_ + st * TILE;
#pragma unroll
    for (int ks = 0; ks < MM_KS; ks += 16) {
      // operands by ldmatrix: the warp's 16 rows of A in one instruction, two groups of 8 columns of W in one
      unsigned a[4];
      mm_ldmatrix_x4(a, As + (warp * 16 + (lane & 15)) * MM_LD + ks + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        unsigned b[4];
        const int off = ((j + (lane >> 4)) * 8 + (lane & 7)) * MM_LD + ks + ((lane >> 3) & 1) * 8;
        mm_ldmatrix_x4(b, B1 + off);
        mma_bf16_16816(c1[j], a, b);
        mma_bf16_16816(c1[j + 1], a, b + 2);
        if (GATED) {
          mm_ldmatrix_x4(b, B2 + off);
          mma_bf16_16816(c2[j], a, b);
          mma_bf16_16816(c2[j + 1], a, b + 2);
        }
      }
    }
    __syncthreads();                               // this stage has been read: the step after next may overwrite it
  }
#pragma unroll
  for (int j = 0; j < 8; j++)
#pragma unroll
    for (int q = 0; q < 4; q++) {
      int r = warp * 16 + g + (q >> 1) * 8, n = n0 + j * 8 + 2 * tq + (q & 1);
      if (r < rows && n < N) {
        const float sc = in_scale ? in_scale[pair_at[row0 + r]] : 1.0f;
        float v = c1[j][q] * sc;
        if (GATED) v = moe_gated(v, c2[j][q] * sc, act);
        out[(size_t)(row0 + r) * N + n] = from_float<TO>(v);
      }
    }
}

// ----------------------------------------------------------------------------- combine
// out[t, :] = sum_k wt[t, k] * y[place[t * top + k], :] + sgate[t] * sum_p shared[p, t, :]   (float32 out)
// A pair whose expert index is E_real or more is an identity expert: its output is the token's input h[t, :].
// sgate may be null: the shared expert then counts in full.
template <typename TS, typename TH>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wt, int top,
                   const TS* __restrict__ shared, int n_parts, size_t part_stride, const float* __restrict__ sgate,
                   float* __restrict__ out, int D, const int* __restrict__ idx, int E_real, const TH* __restrict__ h) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  __shared__ int s_row[MOE_MAX_TOP];            // the pair's row of y, or -1 for an identity expert
  __shared__ float s_wt[MOE_MAX_TOP];
  if (threadIdx.x < top) {
    const size_t p = (size_t)t * top + threadIdx.x;
    s_row[threadIdx.x] = (idx && idx[p] >= E_real) ? -1 : place[p];
    s_wt[threadIdx.x] = wt ? wt[p] : 1.0f;          // no weights: the pairs' outputs are added as they are
  }
  __syncthreads();
  const float sg = (shared && sgate) ? sgate[t] : 1.0f;
  // gridDim.y CTAs share a token's row: few tokens still fill the multiprocessors
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < D; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
#pragma unroll 4
    for (int k = 0; k < top; k++) {
      const int row = s_row[k];
      const float v = row < 0 ? to_float(h[(size_t)t * D + i]) : y[(size_t)row * D + i];
      acc = fmaf(s_wt[k], v, acc);
    }
    if (shared) {
      float s = to_float(shared[(size_t)t * D + i]);
      for (int p = 1; p < n_parts; p++) s += to_float(shared[p * part_stride + (size_t)t * D + i]);
      acc = fmaf(sg, s, acc);
    }
    out[(size_t)t * D + i] = acc;
  }
}

// ----------------------------------------------------------------------------- launchers
// The choice alone, from float32 logits [T, E] that a product left (the thread-per-token form overwrites them).
extern "C" int qd_moe_topk(float* logits, int T, int E, int top, int mode, const float* corr, int* idx, float* wt,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top < 1 || top > E || top > MOE_MAX_TOP) return QD_ERR_UNSUPPORTED;
  if (E <= 32 * MT_PER_LANE)
    qd_launch(moe_topk_warp_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, (const float*)logits, T, E, top, mode, corr,
              idx, wt);
  else
    qd_launch(moe_topk_kernel, dim3((T + 127) / 128), dim3(128), 0, stream, logits, T, E, top, mode, corr, idx, wt);
  return qd_last_error();
}

// logits: float32 scratch [T, E] (left with the chosen entries at -inf)
extern "C" int qd_moe_route(const void* h, const void* wr, const float* br, const void* wsg, int dtype, int T, int D,
                            int E, int top, int mode, const float* corr, float* logits, int* idx, float* wt,
                            float* sgate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top < 1 || top > E || top > MOE_MAX_TOP) return QD_ERR_UNSUPPORTED;
  const int rows = E + (wsg ? 1 : 0);
  dim3 grid((T + MR_TOKENS - 1) / MR_TOKENS, (rows + 7) / 8);
  if (grid.y > 65535) return QD_ERR_UNSUPPORTED;
  const bool al = !(((uintptr_t)h | (uintptr_t)wr | (uintptr_t)wsg) & 15);
#define MR_GO(T_, V_)                                                                                              \
  qd_launch(moe_logits_kernel<T_, V_>, grid, dim3(256), 0, stream, (const T_*)h, (const T_*)wr, br, (const T_*)wsg, T, D, \
            E, logits, sgate)
  if (dtype == QD_F32) { if (al && D % 4 == 0) MR_GO(float, true); else MR_GO(float, false); }
  else if (dtype == QD_BF16) { if (al && D % 8 == 0) MR_GO(bf16, true); else MR_GO(bf16, false); }
  else return QD_ERR_UNSUPPORTED;
#undef MR_GO
  return qd_moe_topk(logits, T, E, top, mode, corr, idx, wt, stream);
}

extern "C" int qd_moe_sort(const int* idx, int n_pairs, int E, int E_real, int tile_rows, int max_tiles, int* place,
                           int* pair_at, int* meta, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (E > 4096) return QD_ERR_UNSUPPORTED;
  qd_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, idx, n_pairs, E, E_real,
            tile_rows, max_tiles, place, pair_at, meta);
  return qd_last_error();
}

// gated != 0: out[place, N] = silu(A W1_e^T) * (A W2_e^T) in ``out_dtype``; else out = A W1_e^T.  in_scale (float32, one
// per pair, or null): the sums of pair p are multiplied by in_scale[p] before the gate.
extern "C" int qd_moe_gemm(const void* A, long long lda, int a_dtype, const int* pair_at, int top, int by_token,
                           const void* W1, const void* W2, int w_dtype, void* out, int out_dtype, int N, int K,
                           const int* meta, int E, int tile_rows, int max_tiles, int gated, int act_kind, float act_limit,
                           float act_alpha, const float* in_scale, cudaStream_t stream) {
  const MoeAct act = {act_kind, act_limit, act_alpha};
  if (max_tiles <= 0) return 0;
  if (max_tiles > 65535 || (tile_rows != 8 && tile_rows != 16 && tile_rows != 64)) return QD_ERR_UNSUPPORTED;
  dim3 grid((N + 63) / 64, max_tiles);
  const bool al16 = !(((uintptr_t)A | (uintptr_t)W1 | (uintptr_t)W2) & 15);
  if (tile_rows == 8) {
    // few rows per expert: the weight-streaming kernel (16-byte pieces: K and the row pitch of A in whole pieces)
    const int es = a_dtype == QD_F32 ? 4 : 2, per = 16 / es;
    size_t smem = (size_t)MG_ROWS * K * es;
    if (!al16 || K % per || lda % per || smem > 200 * 1024) return QD_ERR_UNSUPPORTED;
#define MG_GO(TI, TW, TO, G)                                                                                         \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(moe_gemv_kernel<TI, TW, TO, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    qd_launch(moe_gemv_kernel<TI, TW, TO, G>, grid, dim3(256), smem, stream, (const TI*)A, lda, pair_at, top, by_token, \
              (const TW*)W1, (const TW*)W2, (TO*)out, N, K, meta, E, act, in_scale);                                      \
  } while (0)
#define MG_PICK(TI, TW, TO) do { if (gated) MG_GO(TI, TW, TO, true); else MG_GO(TI, TW, TO, false); } while (0)
    if (a_dtype == QD_F32 && w_dtype == QD_F32 && out_dtype == QD_F32) MG_PICK(float, float, float);
    else if (a_dtype == QD_BF16 && w_dtype == QD_BF16 && out_dtype == QD_BF16) MG_PICK(bf16, bf16, bf16);
    else if (a_dtype == QD_BF16 && w_dtype == QD_BF16 && out_dtype == QD_F32) MG_PICK(bf16, bf16, float);
    else return QD_ERR_UNSUPPORTED;
#undef MG_PICK
#undef MG_GO
    return qd_last_error();
  }
  if (tile_rows == 64 && a_dtype == QD_BF16 && w_dtype == QD_BF16 && al16 && K % 8 == 0 && lda % 8 == 0) {
    // many rows per expert in bfloat16: tensor cores
#define MM_GO(TO, G)                                                                                              \
  do {                                                                                                            \
    const size_t smem = (size_t)(G ? 3 : 2) * 2 * 64 * MM_LD * sizeof(bf16);                                      \
    static bool raised = false;                                                                                   \
    if (!raised && smem > 48 * 1024) {                                                                            \
      cudaFuncSetAttribute(moe_gemm_mma_kernel<TO, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      raised = true;                                                                                              \
    }                                                                                                             \
    qd_launch(moe_gemm_mma_kernel<TO, G>, grid, dim3(128), smem, stream, (const bf16*)A, lda, pair_at, top, by_token, \
              (const bf16*)W1, (const bf16*)W2, (TO*)out, N, K, meta, E, act, in_scale);                          \
  } while (0)
    if (out_dtype == QD_BF16) { if (gated) MM_GO(bf16, true); else MM_GO(bf16, false); }
    else if (out_dtype == QD_F32) { if (gated) MM_GO(float, true); else MM_GO(float, false); }
    else return QD_ERR_UNSUPPORTED;
#undef MM_GO
    return qd_last_error();
  }
#define MOE_GO(TI, TW, TO, TM, G)                                                                                   \
  qd_launch(moe_gemm_kernel<TI, TW, TO, TM, G>, grid, dim3(256), 0, stream, (const TI*)A, lda, pair_at, top, by_token, \
            (const TW*)W1, (const TW*)W2, (TO*)out, N, K, meta, E, act, in_scale)
#define MOE_PICK(TI, TW, TO)                                                     \
  do {                                                                           \
    if (tile_rows == 16) { if (gated) MOE_GO(TI, TW, TO, 16, true); else MOE_GO(TI, TW, TO, 16, false); } \
    else { if (gated) MOE_GO(TI, TW, TO, 64, true); else MOE_GO(TI, TW, TO, 64, false); }                 \
  } while (0)
  if (a_dtype == QD_F32 && w_dtype == QD_F32 && out_dtype == QD_F32) MOE_PICK(float, float, float);
  else if (a_dtype == QD_BF16 && w_dtype == QD_BF16 && out_dtype == QD_BF16) MOE_PICK(bf16, bf16, bf16);
  else if (a_dtype == QD_BF16 && w_dtype == QD_BF16 && out_dtype == QD_F32) MOE_PICK(bf16, bf16, float);
  else return QD_ERR_UNSUPPORTED;
#undef MOE_PICK
#undef MOE_GO
  return qd_last_error();
}

extern "C" int qd_moe_combine(const float* y, const int* place, const float* wt, int top, const void* shared,
                              int shared_dtype, int n_parts, long long part_stride, const float* sgate, float* out,
                              int T, int D, const int* idx, int E_real, const void* h, int h_dtype,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!h) idx = nullptr;
  const int per_row = T >= 1024 ? 1 : (D + 255) / 256 < 16 ? (D + 255) / 256 : 16;
#define MC_GO(TS, TH, NP, PS)                                                                                      \
  qd_launch(moe_combine_kernel<TS, TH>, dim3(T, per_row), dim3(256), 0, stream, y, place, wt, top, (const TS*)shared, NP, \
            (size_t)(PS), sgate, out, D, idx, E_real, (const TH*)h)
  const bool hb = h && h_dtype == QD_BF16;
  if (h && h_dtype != QD_BF16 && h_dtype != QD_F32) return QD_ERR_UNSUPPORTED;
  if (shared && shared_dtype == QD_BF16 && n_parts == 1) {
    if (hb) MC_GO(bf16, bf16, 1, 0); else MC_GO(bf16, float, 1, 0);
  } else if (!shared || shared_dtype == QD_F32) {
    if (hb) MC_GO(float, bf16, n_parts, part_stride); else MC_GO(float, float, n_parts, part_stride);
  } else
    return QD_ERR_UNSUPPORTED;
#undef MC_GO
  return qd_last_error();
}
