// Row-wise kernels of layers that are not the pre-norm RMSNorm/SwiGLU kind:
//
//   tanh norm    out = tanh(alpha * x) * w + b, a norm without statistics; one launch adds what is pending on the
//                residual sum first (one or two branch outputs, each [T, D] or float32 partial sums [n, T, D]; a
//                pending output may be one that joins as unit(y) * u, unit(y) = y / sqrt(mean(y^2) + eps)), writes
//                the sum back, and may write a second norm of the same row (two branches that read the same x)
//                (no norm asked for: the additions alone); it may also write the new sum as a rounded copy
//   gated act    out = act(gate, up) of a stacked [T, 2F] product: silu(g) * u, or the clamped form
//                min(g, L) * sigmoid(a min(g, L)) * (clamp(u, -L, L) + 1)
//   token gate   out = gelu_tanh(z) * table[token, :], a per-token row of a side table gating a small projection
//
// Everything is float32 inside; a row's sums are taken in an order that depends on the row's length only.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float ld_code(const void* p, int code, size_t i) {
  return code == QD_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void st_code(void* p, int code, size_t i, float v) {
  if (code == QD_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
}

// One pending addend of the residual sum.
struct Addend {
  const void* p;        // [n_parts, T, D] (n_parts 1: [T, D]); null: none
  int dtype, n_parts;
  const float* unit_w;  // not null: the addend joins as p / sqrt(mean(p^2) + unit_eps) * unit_w[i]
  float unit_eps;
  float mult;           // the addend (after its unit norm, if any) is multiplied by this constant
};

__device__ __forceinline__ float addend_at(const Addend& a, size_t stride, size_t i) {
  float v = ld_code(a.p, a.dtype, i);
  for (int q = 1; q < a.n_parts; q++) v += ld_code(a.p, a.dtype, q * stride + i);
  return v;
}

struct TanhNorm {
  const float *w, *b;   // [D]
  float alpha;
  void* out;            // [n_rows, D]; null: this norm is not computed
  int out_dtype;
  int rms;              // 1: out = v / sqrt(mean(v^2) + eps) * w instead (b and alpha unused)
  float eps;
};
__device__ __forceinline__ float row_norm(const TanhNorm& n, float v, int i, float fr) {
  return n.rms ? v * fr * n.w[i] : fmaf(tanhf(n.alpha * v), n.w[i], n.b[i]);
}

// One CTA per output row r (source row s = rows[r] or r): v = x[s] + a0[s] + a1[s]; x[s] = v when write_back;
// each norm with an ``out`` writes tanh(alpha v) w + b.
__global__ void __launch_bounds__(256)
add_tanh_norm_kernel(float* __restrict__ x, Addend a0, Addend a1, TanhNorm n0, TanhNorm n1,
                     const int* __restrict__ rows, int D, size_t stride, int write_back, void* __restrict__ copy_out,
                     int copy_dtype) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float f0 = 1.f, f1 = 1.f;
  if (a0.p && a0.unit_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { float v = addend_at(a0, stride, s * D + i); ss = fmaf(v, v, ss); }
    f0 = 1.0f / sqrtf(block_sum(ss, scratch) / (float)D + a0.unit_eps);
  }
  if (a1.p && a1.unit_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { float v = addend_at(a1, stride, s * D + i); ss = fmaf(v, v, ss); }
    f1 = 1.0f / sqrtf(block_sum(ss, scratch) / (float)D + a1.unit_eps);
  }
  f0 *= a0.mult;
  f1 *= a1.mult;
  const bool need_rms = (n0.out && n0.rms) || (n1.out && n1.rms);
  float ssv = 0.f;
  // the new sum: a thread computes the same elements in both passes, in the same way
  auto sum_at = [&](int i) {
    float v = x[s * D + i];
    if (a0.p) { float d = addend_at(a0, stride, s * D + i); v += a0.unit_w ? d * f0 * a0.unit_w[i] : d * f0; }
    if (a1.p) { float d = addend_at(a1, stride, s * D + i); v += a1.unit_w ? d * f1 * a1.unit_w[i] : d * f1; }
    return v;
  };
  if (need_rms) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) { const float v = sum_at(i); ssv = fmaf(v, v, ssv); }
    ssv = block_sum(ssv, scratch);
  }
  const float fr0 = 1.0f / sqrtf(ssv / (float)D + n0.eps), fr1 = 1.0f / sqrtf(ssv / (float)D + n1.eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = sum_at(i);
    if (write_back) x[s * D + i] = v;
    if (copy_out) st_code(copy_out, copy_dtype, (size_t)r * D + i, v);
    if (n0.out) st_code(n0.out, n0.out_dtype, (size_t)r * D + i, row_norm(n0, v, i, fr0));
    if (n1.out) st_code(n1.out, n1.out_dtype, (size_t)r * D + i, row_norm(n1, v, i, fr1));
  }
}

// The same with 16-byte accesses and every operand of a row fetched once, up front, into registers (so that a
// unit-normalised addend costs no second pass): D a multiple of 4 up to 256 * 4 * VPT, all pointers 16-byte aligned.
__device__ __forceinline__ float4 ld4_code(const void* p, int code, size_t i) {      // elements i .. i+3
  if (code == QD_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void st4_code(void* p, int code, size_t i, float4 v) {
  if (code == QD_F32) { *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v; return; }
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&lo);
  raw.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p) + i) = raw;
}
__device__ __forceinline__ float4 addend4_at(const Addend& a, size_t stride, size_t i) {
  float4 v = ld4_code(a.p, a.dtype, i);
  for (int q = 1; q < a.n_parts; q++) {
    const float4 u = ld4_code(a.p, a.dtype, q * stride + i);
    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
  }
  return v;
}
__device__ __forceinline__ float4 tanh_norm4(const TanhNorm& n, float4 v, int i, float fr) {
  const float4 w = *reinterpret_cast<const float4*>(n.w + i);
  if (n.rms) return make_float4(v.x * fr * w.x, v.y * fr * w.y, v.z * fr * w.z, v.w * fr * w.w);
  const float4 b = *reinterpret_cast<const float4*>(n.b + i);
  return make_float4(fmaf(tanhf(n.alpha * v.x), w.x, b.x), fmaf(tanhf(n.alpha * v.y), w.y, b.y),
                     fmaf(tanhf(n.alpha * v.z), w.z, b.z), fmaf(tanhf(n.alpha * v.w), w.w, b.w));
}

template <int VPT>
__global__ void __launch_bounds__(256)
add_tanh_norm_vec_kernel(float* __restrict__ x, Addend a0, Addend a1, TanhNorm n0, TanhNorm n1,
                         const int* __restrict__ rows, int D, size_t stride, int write_back, void* __restrict__ copy_out,
                         int copy_dtype) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float4 xv[VPT], d0[VPT], d1[VPT];
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    const int i = (threadIdx.x + k * 256) * 4;
    xv[k] = d0[k] = d1[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < D) {
      xv[k] = *reinterpret_cast<const float4*>(x + s * D + i);
      if (a0.p) d0[k] = addend4_at(a0, stride, s * D + i);
      if (a1.p) d1[k] = addend4_at(a1, stride, s * D + i);
      ss0 += d0[k].x * d0[k].x + d0[k].y * d0[k].y + d0[k].z * d0[k].z + d0[k].w * d0[k].w;
      ss1 += d1[k].x * d1[k].x + d1[k].y * d1[k].y + d1[k].z * d1[k].z + d1[k].w * d1[k].w;
    }
  }
  float f0 = 1.f, f1 = 1.f;
  if (a0.p && a0.unit_w) f0 = 1.0f / sqrtf(block_sum(ss0, scratch) / (float)D + a0.unit_eps);
  if (a1.p && a1.unit_w) f1 = 1.0f / sqrtf(block_sum(ss1, scratch) / (float)D + a1.unit_eps);
  f0 *= a0.mult;
  f1 *= a1.mult;
  float ssv = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    const int i = (threadIdx.x + k * 256) * 4;
    if (i >= D) continue;
    float4 v = xv[k];
    if (a0.p) {
      float4 d = d0[k];
      if (a0.unit_w) {
        const float4 u = *reinterpret_cast<const float4*>(a0.unit_w + i);
        d = make_float4(d.x * f0 * u.x, d.y * f0 * u.y, d.z * f0 * u.z, d.w * f0 * u.w);
      } else
        d = make_float4(d.x * f0, d.y * f0, d.z * f0, d.w * f0);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    if (a1.p) {
      float4 d = d1[k];
      if (a1.unit_w) {
        const float4 u = *reinterpret_cast<const float4*>(a1.unit_w + i);
        d = make_float4(d.x * f1 * u.x, d.y * f1 * u.y, d.z * f1 * u.z, d.w * f1 * u.w);
      } else
        d = make_float4(d.x * f1, d.y * f1, d.z * f1, d.w * f1);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    xv[k] = v;
    ssv += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    if (write_back) *reinterpret_cast<float4*>(x + s * D + i) = v;
    if (copy_out) st4_code(copy_out, copy_dtype, (size_t)r * D + i, v);
  }
  if ((n0.out && n0.rms) || (n1.out && n1.rms)) ssv = block_sum(ssv, scratch);
  const float fr0 = 1.0f / sqrtf(ssv / (float)D + n0.eps), fr1 = 1.0f / sqrtf(ssv / (float)D + n1.eps);
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    const int i = (threadIdx.x + k * 256) * 4;
    if (i >= D) continue;
    if (n0.out) st4_code(n0.out, n0.out_dtype, (size_t)r * D + i, tanh_norm4(n0, xv[k], i, fr0));
    if (n1.out) st4_code(n1.out, n1.out_dtype, (size_t)r * D + i, tanh_norm4(n1, xv[k], i, fr1));
  }
}

// x [T, D] float32 (updated when write_back).  Addend k: ak [nk, T, D] of dtype code ak_dtype, null for none; with
// ak_unit_w it joins unit-normalised.  Norm k: wk, bk [D] float32, alphak, outk [n_rows, D] (null: not computed).
// An addend is multiplied by its ``mult``; a norm with ``rms`` set is out = v / sqrt(mean(v^2) + eps) * w instead.
// rows: int32 [n_rows] source rows, or null for all T rows in order.  copy_out [n_rows, D]: the new sum itself in
// dtype copy_dtype (null: not written).
extern "C" int qd_add_tanh_norm(float* x, int T, int D,
                                const void* a0, int a0_dtype, int a0_parts, const float* a0_unit_w, float a0_eps, float a0_mult,
                                const void* a1, int a1_dtype, int a1_parts, const float* a1_unit_w, float a1_eps, float a1_mult,
                                const float* w0, const float* b0, float alpha0, void* out0, int out0_dtype, int rms0, float eps0,
                                const float* w1, const float* b1, float alpha1, void* out1, int out1_dtype, int rms1, float eps1,
                                const int* rows, int n_rows, int write_back, void* copy_out, int copy_dtype,
                                cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  Addend A0 = {a0, a0_dtype, a0_parts, a0_unit_w, a0_eps, a0_mult}, A1 = {a1, a1_dtype, a1_parts, a1_unit_w, a1_eps, a1_mult};
  TanhNorm N0 = {w0, b0, alpha0, out0, out0_dtype, rms0, eps0}, N1 = {w1, b1, alpha1, out1, out1_dtype, rms1, eps1};
  const uintptr_t all = (uintptr_t)x | (uintptr_t)a0 | (uintptr_t)a1 | (uintptr_t)a0_unit_w | (uintptr_t)a1_unit_w |
                        (uintptr_t)w0 | (uintptr_t)b0 | (uintptr_t)out0 | (uintptr_t)w1 | (uintptr_t)b1 |
                        (uintptr_t)out1 | (uintptr_t)copy_out;
#define TN_GO(K)                                                                                                   \
  qd_launch(K, dim3(n_rows), dim3(256), 0, stream, x, A0, A1, N0, N1, rows, D, (size_t)T * D, write_back, copy_out, \
            copy_dtype)
  if (D % 4 == 0 && !(all & 15) && D <= 256 * 4 * 4) {
    if (D <= 256 * 4) TN_GO(add_tanh_norm_vec_kernel<1>);
    else if (D <= 256 * 8) TN_GO(add_tanh_norm_vec_kernel<2>);
    else TN_GO(add_tanh_norm_vec_kernel<4>);
  } else
    TN_GO(add_tanh_norm_kernel);
#undef TN_GO
  return qd_last_error();
}

// ------------------------------------------------------------------------------------------------ gated activation
__global__ void __launch_bounds__(256)
gated_act_kernel(const void* __restrict__ gu, int in_dtype, void* __restrict__ out, int out_dtype, int F, size_t n,
                 int kind, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / F, f = i - t * F;
    float g = ld_code(gu, in_dtype, t * 2 * F + f), u = ld_code(gu, in_dtype, t * 2 * F + F + f);
    float v;
    if (kind == 0) v = g / (1.0f + expf(-g)) * u;
    else {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      v = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    }
    st_code(out, out_dtype, i, v);
  }
}

// Four elements per thread with 16-byte (float32) or 8-byte (bfloat16) accesses: F a multiple of 4, aligned pointers.
__device__ __forceinline__ float gated_one(float g, float u, int kind, float limit, float alpha) {
  if (kind == 0) return g / (1.0f + expf(-g)) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}
__global__ void __launch_bounds__(256)
gated_act_vec_kernel(const void* __restrict__ gu, int in_dtype, void* __restrict__ out, int out_dtype, int F4, size_t n4,
                     int kind, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / F4, f = (i - t * F4) * 4;
    const float4 g = ld4_code(gu, in_dtype, t * 8 * F4 + f), u = ld4_code(gu, in_dtype, t * 8 * F4 + 4 * (size_t)F4 + f);
    st4_code(out, out_dtype, i * 4, make_float4(gated_one(g.x, u.x, kind, limit, alpha), gated_one(g.y, u.y, kind, limit, alpha),
                                                gated_one(g.z, u.z, kind, limit, alpha), gated_one(g.w, u.w, kind, limit, alpha)));
  }
}

extern "C" int qd_gated_act(const void* gate_up, int in_dtype, void* out, int out_dtype, int T, int F, int kind,
                            float limit, float alpha, cudaStream_t stream) {
  const size_t n = (size_t)T * F;
  if (n == 0) return 0;
  if (F % 4 == 0 && !(((uintptr_t)gate_up | (uintptr_t)out) & 15)) {
    const size_t n4 = n / 4;
    unsigned blocks = (unsigned)((n4 + 255) / 256 < 65535 ? (n4 + 255) / 256 : 65535);
    qd_launch(gated_act_vec_kernel, dim3(blocks), dim3(256), 0, stream, gate_up, in_dtype, out, out_dtype, F / 4, n4, kind,
              limit, alpha);
    return qd_last_error();
  }
  unsigned blocks = (unsigned)((n + 255) / 256 < 65535 ? (n + 255) / 256 : 65535);
  qd_launch(gated_act_kernel, dim3(blocks), dim3(256), 0, stream, gate_up, in_dtype, out, out_dtype, F, n, kind, limit,
            alpha);
  return qd_last_error();
}

// ------------------------------------------------------------------------------------------------ token gate
// out[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], j]
__global__ void __launch_bounds__(256)
token_gate_kernel(const void* __restrict__ z, int z_dtype, const void* __restrict__ table, int table_dtype,
                  const int* __restrict__ tokens, void* __restrict__ out, int out_dtype, int W, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / W, j = i - t * W;
    const float v = ld_code(z, z_dtype, i);
    const float g = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    st_code(out, out_dtype, i, g * ld_code(table, table_dtype, (size_t)tokens[t] * W + j));
  }
}

extern "C" int qd_token_gate(const void* z, int z_dtype, const void* table, int table_dtype, const int* tokens,
                             void* out, int out_dtype, int T, int W, cudaStream_t stream) {
  const size_t n = (size_t)T * W;
  if (n == 0) return 0;
  unsigned blocks = (unsigned)((n + 255) / 256 < 65535 ? (n + 255) / 256 : 65535);
  qd_launch(token_gate_kernel, dim3(blocks), dim3(256), 0, stream, z, z_dtype, table, table_dtype, tokens, out,
            out_dtype, W, n);
  return qd_last_error();
}
