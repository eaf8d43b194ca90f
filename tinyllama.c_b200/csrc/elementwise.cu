// Embedding gather, RMSNorm, gated grouped RMSNorm and the SwiGLU product.
//
// Math follows CodeClaper/tinyllama.c's CPU ops: embedding row gather (cpu_op.c:508-524),
// RMSNorm ss=sum x^2, s=1/sqrt(ss/n+eps), o=x*s*w (cpu_op.c:44-64), SiLU x/(1+exp(-x))
// (cpu_op.c:332-335), the Mamba2 gate and grouped norm (cpu_op.c:950-958).  All
// statistics are 32-bit; only the stored result takes the activation type.
#include "common.cuh"
#include <stdarg.h>

int g_tlc_pdl = 0;
extern "C" void tlc_set_pdl(int on) { g_tlc_pdl = on; }

static thread_local char g_err[512];
extern "C" const char* tlc_last_error() { return g_err; }
int tlc_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// ---- embedding ---------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, int D, int V,
                             float scale, float* __restrict__ out) {
  tlc_pdl(tokens, out);
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);   // ids are validated on the host; never read out of bounds
  const TW* row = table + (size_t)tok * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[(size_t)t * D + d] = to_f32(row[d]) * scale;
}

extern "C" int tlc_embed(const int* tokens, const void* table, int table_dtype, int T, int D, int V, float scale,
                         float* out, cudaStream_t stream) {
  if (T == 0) return 0;
  // the first kernel of a step: a full dependency on everything before it (see tlc_launch_step_boundary)
  TLC_DISPATCH_DTYPE(table_dtype, TW, tlc_launch_step_boundary(embed_kernel<TW>, dim3(T), dim3(256), 0, stream, tokens,
                                                               (const TW*)table, D, V, scale, out));
  TLC_CHECK_LAUNCH("embed");
  return 0;
}

// ---- RMSNorm of 32-bit rows ----------------------------------------------------------
// One block per row.  The row stays in registers between the sum of squares and the scaling
// when it fits (up to RMS_MAX_PER_THREAD values per thread), otherwise it is read twice.
#define RMS_MAX_PER_THREAD 16
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, int x_ld, const int* __restrict__ rows, const float* __restrict__ w,
               float eps, int D, TO* __restrict__ out) {
  tlc_pdl(x, rows, out);
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * x_ld;
  float ss = 0.f;
  if (D <= 256 * RMS_MAX_PER_THREAD) {
    float v[RMS_MAX_PER_THREAD];
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      v[i] = d < D ? xr[d] : 0.f;
      ss += v[i] * v[i];
    }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      if (d < D) out[(size_t)r * D + d] = from_f32<TO>(v[i] * s * w[d]);
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) { float v = xr[d]; ss += v * v; }
  ss = block_sum(ss, red);
  const float s = 1.0f / sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[(size_t)r * D + d] = from_f32<TO>(xr[d] * s * w[d]);
}

// Rows whose width is a multiple of 4 (up to 16384): NT threads take PT float4 each.  The weight
// does not depend on the kernel before this one and is fetched before the wait on it.  NT and PT
// follow from the width alone, so a row's sum has the same tree whatever else is in the batch.
template <typename TO> struct Out4;
template <> struct Out4<float> {
  static __device__ __forceinline__ void put(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  }
};
template <> struct Out4<__nv_bfloat16> {
  static __device__ __forceinline__ void put(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

// element i (or the four from i on) of a buffer whose type is known at run time
__device__ __forceinline__ void put_as(void* p, int dtype, size_t i, float v) {
  if (dtype == TLC_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
  else reinterpret_cast<float*>(p)[i] = v;
}
__device__ __forceinline__ void put4_as(void* p, int dtype, size_t i, float4 v) {
  if (dtype == TLC_BF16) Out4<__nv_bfloat16>::put(reinterpret_cast<__nv_bfloat16*>(p) + i, v.x, v.y, v.z, v.w);
  else Out4<float>::put(reinterpret_cast<float*>(p) + i, v.x, v.y, v.z, v.w);
}

template <typename TO, int NT, int PT>
__global__ void __launch_bounds__(NT)
rmsnorm_vec_kernel(const float* __restrict__ x, int x_ld, const int* __restrict__ rows, const float* __restrict__ w,
                   float eps, int D, TO* __restrict__ out) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[33];
  const int n4 = D >> 2;
  float4 wv[PT], v[PT];
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    wv[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(w) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tlc_wait(x, rows, out);
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * x_ld);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < PT; i++) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  ss = block_sum(ss, red);
  const float s = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c < n4)
      Out4<TO>::put(out + (size_t)r * D + 4 * c, v[i].x * s * wv[i].x, v[i].y * s * wv[i].y, v[i].z * s * wv[i].z,
                    v[i].w * s * wv[i].w);
  }
}

// picks NT, PT from the number of float4 in a row (at most 4096 of them)
#define TLC_VEC_SHAPES(n4, LAUNCH)            \
  if ((n4) <= 128) { LAUNCH(128, 1); }        \
  else if ((n4) <= 256) { LAUNCH(256, 1); }   \
  else if ((n4) <= 512) { LAUNCH(512, 1); }   \
  else if ((n4) <= 1024) { LAUNCH(1024, 1); } \
  else if ((n4) <= 2048) { LAUNCH(1024, 2); } \
  else { LAUNCH(1024, 4); }

// The same for many rows (prompts): fewer threads a row with up to four float4 each, so that a thread has more
// loads in flight, more rows share an SM, and the block's sum has fewer warps to join.
#define TLC_VEC_SHAPES_MANY(n4, LAUNCH)       \
  if ((n4) <= 128) { LAUNCH(64, 2); }         \
  else if ((n4) <= 256) { LAUNCH(64, 4); }    \
  else if ((n4) <= 512) { LAUNCH(128, 4); }   \
  else if ((n4) <= 768) { LAUNCH(256, 3); }   \
  else if ((n4) <= 1024) { LAUNCH(256, 4); }  \
  else if ((n4) <= 2048) { LAUNCH(512, 4); }  \
  else { LAUNCH(1024, 4); }
constexpr int VEC_MANY_ROWS = 512;            // from this many rows on

extern "C" int tlc_rmsnorm(const float* x, int x_ld, const int* rows, const float* w, float eps, int R, int D, void* out,
                           int out_dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  TLC_REQUIRE(x_ld >= D, "rmsnorm: rows of %d values with a stride of %d", D, x_ld);
  if (D % 4 == 0 && x_ld % 4 == 0 && D <= 16384 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    const int n4 = D / 4;
#define TLC_RMS_LAUNCH(NT, PT)                                                                                        \
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(rmsnorm_vec_kernel<TO, NT, PT>, dim3(R), dim3(NT), 0, stream, x, x_ld, rows, w, \
                                               eps, D, (TO*)out))
    if (R >= VEC_MANY_ROWS) { TLC_VEC_SHAPES_MANY(n4, TLC_RMS_LAUNCH) } else { TLC_VEC_SHAPES(n4, TLC_RMS_LAUNCH) }
#undef TLC_RMS_LAUNCH
    TLC_CHECK_LAUNCH("rmsnorm");
    return 0;
  }
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(rmsnorm_kernel<TO>, dim3(R), dim3(256), 0, stream, x, x_ld, rows, w, eps, D, (TO*)out));
  TLC_CHECK_LAUNCH("rmsnorm");
  return 0;
}

// ---- gate and grouped RMSNorm of the scan output ---------------------------------------
// the gate of a normed read-out: SiLU of z, or (sig) its sigmoid alone
__device__ __forceinline__ float gate_f(float z, bool sig) { return sig ? 1.0f / (1.0f + expf(-z)) : silu_f(z); }
template <bool QUICK> __device__ __forceinline__ float gate_of(float z, bool sig) {
  return sig ? (QUICK ? __fdividef(1.0f, 1.0f + __expf(-z)) : 1.0f / (1.0f + expf(-z))) : silu_of<QUICK>(z);
}
// y [T, Di] 32-bit; z a strided slice of the input projection; out rows of out_ld elements, the whole
// result times out_scale; one block per (row, group).
template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ y2, const TZ* __restrict__ z, int ldz,
                                     const float* __restrict__ w, float eps, int Di, int gs, int mode,
                                     TO* __restrict__ out, int out_ld, float out_scale) {
  tlc_pdl(y, y2, z, out);
  __shared__ float red[33];
  const bool norm_before_gate = mode & TLC_GATE_NORM_FIRST, sig = mode & TLC_GATE_SIGMOID;
  const int t = blockIdx.x, g = blockIdx.y;
  const float* yr = y + (size_t)t * Di + (size_t)g * gs;
  const float* y2r = y2 ? y2 + (size_t)t * Di + (size_t)g * gs : nullptr;    // a second summand of the input
  const TZ* zr = z + (size_t)t * ldz + (size_t)g * gs;
  TO* o = out + (size_t)t * out_ld + (size_t)g * gs;
  if (w == nullptr) {                                   // no norm: y * silu(z)
    for (int d = threadIdx.x; d < gs; d += blockDim.x) o[d] = from_f32<TO>((yr[d] + (y2r ? y2r[d] : 0.f)) * gate_f(to_f32(zr[d]), sig) * out_scale);
    return;
  }
  const float* wg = w + (size_t)g * gs;
  float ss = 0.f;
  if (gs <= 256 * RMS_MAX_PER_THREAD) {
    // one pass: y and the gate are read once; what is normalised stays in registers
    float v[RMS_MAX_PER_THREAD], gate[RMS_MAX_PER_THREAD];
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {          // every load is issued before the first exp
      const int d = threadIdx.x + i * 256;
      gate[i] = d < gs ? to_f32(zr[d]) : 0.f;
      v[i] = d < gs ? yr[d] + (y2r ? y2r[d] : 0.f) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      gate[i] = gate_f(gate[i], sig);
      if (!norm_before_gate) v[i] *= gate[i];
      ss += v[i] * v[i];
    }
    ss = block_sum(ss, red);
    const float s = out_scale / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      if (d < gs) o[d] = from_f32<TO>(norm_before_gate ? (v[i] * s * wg[d]) * gate[i] : v[i] * s * wg[d]);
    }
    return;
  }
  for (int d = threadIdx.x; d < gs; d += blockDim.x) {
    float v = yr[d] + (y2r ? y2r[d] : 0.f);
    if (!norm_before_gate) v *= gate_f(to_f32(zr[d]), sig);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float s = out_scale / sqrtf(ss / (float)gs + eps);
  for (int d = threadIdx.x; d < gs; d += blockDim.x) {
    const float gate = gate_f(to_f32(zr[d]), sig);
    float v = yr[d] + (y2r ? y2r[d] : 0.f);
    v = norm_before_gate ? (v * s * wg[d]) * gate : (v * gate) * s * wg[d];
    o[d] = from_f32<TO>(v);
  }
}

// Groups whose width is a multiple of 4 (up to 16384), 32-bit gate: NT threads take PT float4 each;
// the weight is fetched before the wait on the previous kernel.
template <typename TO, int NT, int PT>
__global__ void __launch_bounds__(NT)
gated_rmsnorm_vec_kernel(const float* __restrict__ y, const float* __restrict__ y2, const float* __restrict__ z, int ldz, const float* __restrict__ w,
                         float eps, int Di, int gs, int mode, TO* __restrict__ out, int out_ld,
                         float out_scale) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[33];
  const bool norm_before_gate = mode & TLC_GATE_NORM_FIRST, sig = mode & TLC_GATE_SIGMOID;
  const int t = blockIdx.x, g = blockIdx.y;
  const int n4 = gs >> 2;
  float4 wv[PT], v[PT], gate[PT];
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    wv[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(w + (size_t)g * gs) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tlc_wait(y, y2, z, out);
  const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * Di + (size_t)g * gs);
  const float4* y2r = y2 ? reinterpret_cast<const float4*>(y2 + (size_t)t * Di + (size_t)g * gs) : nullptr;
  const float4* zr = reinterpret_cast<const float4*>(z + (size_t)t * ldz + (size_t)g * gs);
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    v[i] = c < n4 ? yr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    gate[i] = c < n4 ? zr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (y2r != nullptr && c < n4) {                     // the input comes as two summands
      const float4 u = y2r[c];
      v[i] = make_float4(v[i].x + u.x, v[i].y + u.y, v[i].z + u.z, v[i].w + u.w);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    constexpr bool QUICK = sizeof(TO) == 2;              // a bfloat16 output means a bfloat16 run
    gate[i] = make_float4(gate_of<QUICK>(gate[i].x, sig), gate_of<QUICK>(gate[i].y, sig), gate_of<QUICK>(gate[i].z, sig), gate_of<QUICK>(gate[i].w, sig));
    if (!norm_before_gate) { v[i].x *= gate[i].x; v[i].y *= gate[i].y; v[i].z *= gate[i].z; v[i].w *= gate[i].w; }
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  ss = block_sum(ss, red);
  const float s = out_scale / sqrtf(ss / (float)gs + eps);
  TO* o = out + (size_t)t * out_ld + (size_t)g * gs;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c < n4) {
      if (norm_before_gate)
        Out4<TO>::put(o + 4 * c, (v[i].x * s * wv[i].x) * gate[i].x, (v[i].y * s * wv[i].y) * gate[i].y,
                      (v[i].z * s * wv[i].z) * gate[i].z, (v[i].w * s * wv[i].w) * gate[i].w);
      else
        Out4<TO>::put(o + 4 * c, v[i].x * s * wv[i].x, v[i].y * s * wv[i].y, v[i].z * s * wv[i].z, v[i].w * s * wv[i].w);
    }
  }
}

// Groups of at most 32 float4 (a head of up to 128 values): a warp per group, eight groups a block, the sum by shuffles
// alone.  The shape follows from the group's width alone, so a group's sum has the same tree in every step.
template <typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_warp_kernel(const float* __restrict__ y, const float* __restrict__ y2, const float* __restrict__ z, int ldz,
                          const float* __restrict__ w, float eps, long long n_rows, int n_groups, int Di, int gs,
                          int mode, TO* __restrict__ out, int out_ld, float out_scale) {
  asm volatile("griddepcontrol.launch_dependents;");
  const bool norm_before_gate = mode & TLC_GATE_NORM_FIRST, sig = mode & TLC_GATE_SIGMOID;
  const long long idx = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31, n4 = gs >> 2;
  const bool on = idx < n_rows && lane < n4;
  const long long t = idx / n_groups;
  const int g = (int)(idx % n_groups);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 wv = on ? __ldg(reinterpret_cast<const float4*>(w + (size_t)g * gs) + lane) : zero;
  tlc_wait(y, y2, z, out);
  float4 v = zero, gate = zero;
  if (on) {
    v = reinterpret_cast<const float4*>(y + (size_t)t * Di + (size_t)g * gs)[lane];
    gate = reinterpret_cast<const float4*>(z + (size_t)t * ldz + (size_t)g * gs)[lane];
    if (y2 != nullptr) {
      const float4 u = reinterpret_cast<const float4*>(y2 + (size_t)t * Di + (size_t)g * gs)[lane];
      v = make_float4(v.x + u.x, v.y + u.y, v.z + u.z, v.w + u.w);
    }
  }
  constexpr bool QUICK = sizeof(TO) == 2;                // a bfloat16 output means a bfloat16 run
  gate = make_float4(gate_of<QUICK>(gate.x, sig), gate_of<QUICK>(gate.y, sig), gate_of<QUICK>(gate.z, sig), gate_of<QUICK>(gate.w, sig));
  if (!norm_before_gate) { v.x *= gate.x; v.y *= gate.y; v.z *= gate.z; v.w *= gate.w; }
  const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
  const float s = out_scale / sqrtf(ss / (float)gs + eps);
  if (!on) return;
  TO* o = out + (size_t)t * out_ld + (size_t)g * gs + 4 * lane;
  if (norm_before_gate)
    Out4<TO>::put(o, (v.x * s * wv.x) * gate.x, (v.y * s * wv.y) * gate.y, (v.z * s * wv.z) * gate.z, (v.w * s * wv.w) * gate.w);
  else
    Out4<TO>::put(o, v.x * s * wv.x, v.y * s * wv.y, v.z * s * wv.z, v.w * s * wv.w);
}

extern "C" int tlc_gated_rmsnorm(const float* y, const float* y2, const void* z, int z_dtype, int ldz, const float* w, float eps, int T,
                                 int Di, int n_groups, int mode, void* out, int out_dtype, int out_ld,
                                 float out_scale, cudaStream_t stream) {
  if (T == 0) return 0;
  if (out_ld <= 0) out_ld = Di;                          // elements between rows of out (0: dense)
  TLC_REQUIRE(n_groups > 0 && Di % n_groups == 0, "gated_rmsnorm: width %d is not a multiple of %d groups", Di, n_groups);
  const int gs = Di / n_groups;
  dim3 grid(T, n_groups);
  if (w != nullptr && z_dtype == TLC_F32 && gs % 4 == 0 && gs <= 16384 && ldz % 4 == 0 && ((uintptr_t)y % 16) == 0 &&
      ((uintptr_t)z % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0 && out_ld % 4 == 0 &&
      ((uintptr_t)y2 % 16) == 0) {
    const int n4 = gs / 4;
    if (n4 <= 32) {
      const long long n_rows = (long long)T * n_groups;
      TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(gated_rmsnorm_warp_kernel<TO>, dim3((unsigned)((n_rows + 7) / 8)), dim3(256), 0, stream,
                                                   y, y2, (const float*)z, ldz, w, eps, n_rows, n_groups, Di, gs, mode,
                                                   (TO*)out, out_ld, out_scale));
      TLC_CHECK_LAUNCH("gated_rmsnorm");
      return 0;
    }
#define TLC_GRMS_LAUNCH(NT, PT)                                                                                         \
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(gated_rmsnorm_vec_kernel<TO, NT, PT>, grid, dim3(NT), 0, stream, y, y2,    \
                                               (const float*)z, ldz, w, eps, Di, gs, mode, (TO*)out, out_ld, out_scale))
    if (T >= VEC_MANY_ROWS) { TLC_VEC_SHAPES_MANY(n4, TLC_GRMS_LAUNCH) } else { TLC_VEC_SHAPES(n4, TLC_GRMS_LAUNCH) }
#undef TLC_GRMS_LAUNCH
    TLC_CHECK_LAUNCH("gated_rmsnorm");
    return 0;
  }
  TLC_DISPATCH_DTYPE(z_dtype, TZ, TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(gated_rmsnorm_kernel<TZ, TO>, dim3(grid), dim3(256), 0, stream, 
      y, y2, (const TZ*)z, ldz, w, eps, Di, gs, mode, (TO*)out, out_ld, out_scale)));
  TLC_CHECK_LAUNCH("gated_rmsnorm");
  return 0;
}

// ---- gated product: out = act(gate) * up, gate|up side by side in one row -----------------
// interleave: gate and up come in groups of 16 columns (8 gates, then their 8 ups) instead of as two halves.
// ACT 0: SiLU; 1: the tanh form of GELU, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
template <int ACT> __device__ __forceinline__ float glu_act(float z) { return ACT == 1 ? gelu_tanh_f(z) : silu_f(z); }

template <typename TI, typename T, int ACT>
__global__ void glu_kernel(const TI* __restrict__ gu, int ld, int F, T* __restrict__ out, size_t total, int interleave, float limit,
                           float alpha) {
  tlc_pdl(gu, out);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / F;
  const int f = (int)(i % F);
  const int gc = interleave ? (f >> 3) * 16 + (f & 7) : f, uc = interleave ? gc + 8 : F + f;
  const float g = to_f32(gu[t * ld + gc]), u = to_f32(gu[t * ld + uc]);
  if (ACT == TLC_ACT_SWISH_CLAMPED) out[i] = from_f32<T>(moe_pair_act<false>(ACT, 1, limit, alpha, 1.0f, g, u));
  else out[i] = from_f32<T>(glu_act<ACT>(g) * u);
}

extern "C" int tlc_glu(const void* gu, int in_dtype, int ld, int F, int T, void* out, int dtype, int interleave, int act,
                       float limit, float alpha, cudaStream_t stream) {
  const size_t total = (size_t)T * F;
  if (total == 0) return 0;
  TLC_REQUIRE(act >= 0 && act <= 2, "glu: unknown activation %d (0 SiLU, 1 GELU in its tanh form, 2 the clamped swish)", act);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (act == 2) {
    TLC_DISPATCH_DTYPE(in_dtype, TI, TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(glu_kernel<TI, TT, 2>, dim3(blocks), dim3(256), 0, stream,
        (const TI*)gu, ld, F, (TT*)out, total, interleave, limit, alpha)));
  } else if (act == 1) {
    TLC_DISPATCH_DTYPE(in_dtype, TI, TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(glu_kernel<TI, TT, 1>, dim3(blocks), dim3(256), 0, stream,
        (const TI*)gu, ld, F, (TT*)out, total, interleave, limit, alpha)));
  } else {
    TLC_DISPATCH_DTYPE(in_dtype, TI, TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(glu_kernel<TI, TT, 0>, dim3(blocks), dim3(256), 0, stream,
        (const TI*)gu, ld, F, (TT*)out, total, interleave, limit, alpha)));
  }
  TLC_CHECK_LAUNCH("glu");
  return 0;
}

extern "C" int tlc_swiglu(const void* gu, int in_dtype, int ld, int F, int T, void* out, int dtype, int interleave,
                          cudaStream_t stream) {
  return tlc_glu(gu, in_dtype, ld, F, T, out, dtype, interleave, 0, 0.f, 1.0f, stream);
}

// ---- RMSNorm with token shift --------------------------------------------------------------
// n[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w;  out[t] = n[t] + (n[t-1] - n[t]) * mu, where n[t-1] is the normed row of
// the sequence's previous token: the row above in this step, or what the sequence's slot of `state` [n_slots, D] holds
// from its last step (zeros at position 0).  One block per row; it norms the row above by itself, and the block of a
// sequence's first row of the step, which is the only one to read the slot, afterwards leaves the sequence's last normed
// row there (every thread reads the elements it later writes).
__device__ __forceinline__ float row_inv_rms(const float* xr, int D, float eps, float* red) {
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = xr[d]; ss += v * v; }
  ss = block_sum(ss, red);
  return 1.0f / sqrtf(ss / (float)D + eps);
}

template <typename TO>
__global__ void __launch_bounds__(1024)
rmsnorm_shift_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ mu, float eps, int D,
                     const int* __restrict__ row_seq, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                     const int* __restrict__ start_pos, float* state, TO* __restrict__ out) {
  tlc_pdl(x, state, out);
  __shared__ float red[33];
  const int t = blockIdx.x, b = row_seq[t];
  const int first = cu_seqlens[b], last = cu_seqlens[b + 1] - 1;
  const float* xr = x + (size_t)t * D;
  const float s = row_inv_rms(xr, D, eps, red);
  if (t > first) {
    const float* xp = xr - D;
    const float sp = row_inv_rms(xp, D, eps, red);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const float n = xr[d] * s * w[d], p = xp[d] * sp * w[d];
      out[(size_t)t * D + d] = from_f32<TO>(n + (p - n) * mu[d]);
    }
    return;
  }
  float* st = state + (size_t)slots[b] * D;
  const bool fresh = start_pos[b] == 0;
  const float* xl = x + (size_t)last * D;
  const float sl = last == t ? s : row_inv_rms(xl, D, eps, red);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float n = xr[d] * s * w[d], p = fresh ? 0.f : st[d];
    out[(size_t)t * D + d] = from_f32<TO>(n + (p - n) * mu[d]);
    st[d] = xl[d] * sl * w[d];
  }
}

extern "C" int tlc_rmsnorm_shift(const float* x, const float* w, const float* mu, float eps, int T, int D, const int* row_seq,
                                 const int* cu_seqlens, const int* slots, const int* start_pos, float* state, void* out,
                                 int out_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  const int nt = (T < 256 && D >= 1024) ? 1024 : 256;       // few rows: more threads a row
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(rmsnorm_shift_kernel<TO>, dim3(T), dim3(nt), 0, stream, x, w, mu, eps, D, row_seq,
                                               cu_seqlens, slots, start_pos, state, (TO*)out));
  TLC_CHECK_LAUNCH("rmsnorm_shift");
  return 0;
}

// ---- RMSNorm of a sublayer's output, added into the residual stream ---------------------------
// y[t] = sum over p < n_parts of parts[t, p, :] (in this order) + g[t] * extra[t, :] (where extra is given), with
// g[t] = gate[t * gate_ld], or its sigmoid;  res[t] (+)= y[t] / sqrt(mean(y[t]^2) + eps) * w, or y[t] itself where w is
// NULL.  One block per row; the summed row waits in shared memory for its scale where it fits, else it is summed twice.
__global__ void __launch_bounds__(1024)
rmsnorm_add_kernel(const float* __restrict__ parts, int n_parts, const float* __restrict__ extra,
                   const float* __restrict__ gate, int gate_ld, int gate_sigmoid, const float* __restrict__ w, float eps, int D,
                   float* __restrict__ res, int accumulate, int keep, void* __restrict__ copy, int copy_dtype) {
  tlc_pdl(parts, extra, gate, res, copy);
  __shared__ float red[33];
  extern __shared__ float yrow[];               // the summed row, where it fits (keep)
  const int t = blockIdx.x;
  const float* pr = parts + (size_t)t * n_parts * D;
  const float* er = extra ? extra + (size_t)t * D : nullptr;
  float g = 1.0f;
  if (gate) {
    g = gate[(size_t)t * gate_ld];
    if (gate_sigmoid) g = 1.0f / (1.0f + expf(-g));
  }
  float s = 1.0f;
  if (w) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float y = 0.f;
#pragma unroll 4
      for (int p = 0; p < n_parts; p++) y += pr[(size_t)p * D + d];
      if (er) y = fmaf(g, er[d], y);
      if (keep) yrow[d] = y;
      ss += y * y;
    }
    ss = block_sum(ss, red);
    s = 1.0f / sqrtf(ss / (float)D + eps);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float y;
    if (w && keep) {
      y = yrow[d];                              // (written by this thread)
    } else {
      y = 0.f;
      for (int p = 0; p < n_parts; p++) y += pr[(size_t)p * D + d];
      if (er) y = fmaf(g, er[d], y);
    }
    const float v = w ? y * s * w[d] : y;
    float* o = res + (size_t)t * D + d;
    const float r = accumulate ? *o + v : v;
    *o = r;
    if (copy) put_as(copy, copy_dtype, (size_t)t * D + d, r);
  }
}

// The same with a row in registers: 16-byte loads and stores, the weight fetched before the wait on the previous kernel.
// D a multiple of 4, at most 4 * NT * PT; the sums run in the order of the kernel above.
template <int NT, int PT>
__global__ void __launch_bounds__(NT)
rmsnorm_add_vec_kernel(const float* __restrict__ parts, int n_parts, const float* __restrict__ extra,
                       const float* __restrict__ gate, int gate_ld, int gate_sigmoid, const float* __restrict__ w, float eps,
                       int D, float* __restrict__ res, int accumulate, void* __restrict__ copy, int copy_dtype) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[33];
  const int n4 = D >> 2, t = blockIdx.x;
  float4 wv[PT], v[PT];
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    wv[i] = (w && c < n4) ? __ldg(reinterpret_cast<const float4*>(w) + c) : make_float4(1.f, 1.f, 1.f, 1.f);
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tlc_wait(parts, extra, gate, res, copy);
  const float4* pr = reinterpret_cast<const float4*>(parts + (size_t)t * n_parts * D);
  for (int p = 0; p < n_parts; p++) {
#pragma unroll
    for (int i = 0; i < PT; i++) {
      const int c = threadIdx.x + i * NT;
      if (c < n4) {
        const float4 a = pr[(size_t)p * n4 + c];
        v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
      }
    }
  }
  if (extra) {
    float g = 1.0f;
    if (gate) {
      g = gate[(size_t)t * gate_ld];
      if (gate_sigmoid) g = 1.0f / (1.0f + expf(-g));
    }
    const float4* er = reinterpret_cast<const float4*>(extra + (size_t)t * D);
#pragma unroll
    for (int i = 0; i < PT; i++) {
      const int c = threadIdx.x + i * NT;
      if (c < n4) {
        const float4 a = er[c];
        v[i].x = fmaf(g, a.x, v[i].x); v[i].y = fmaf(g, a.y, v[i].y); v[i].z = fmaf(g, a.z, v[i].z); v[i].w = fmaf(g, a.w, v[i].w);
      }
    }
  }
  float4 r[PT];
  float4* rr = reinterpret_cast<float4*>(res + (size_t)t * D);
#pragma unroll
  for (int i = 0; i < PT; i++) {                           // in flight during the block's sum
    const int c = threadIdx.x + i * NT;
    r[i] = (accumulate && c < n4) ? rr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float s = 1.0f;
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PT; i++) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = block_sum(ss, red);
    s = 1.0f / sqrtf(ss / (float)D + eps);
  }
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c >= n4) continue;
    if (w) {
      r[i].x += v[i].x * s * wv[i].x; r[i].y += v[i].y * s * wv[i].y; r[i].z += v[i].z * s * wv[i].z; r[i].w += v[i].w * s * wv[i].w;
    } else {
      r[i].x += v[i].x; r[i].y += v[i].y; r[i].z += v[i].z; r[i].w += v[i].w;
    }
    rr[c] = r[i];
    if (copy) put4_as(copy, copy_dtype, (size_t)t * D + 4 * c, r[i]);
  }
}

static bool aligned16(const void* p) { return ((uintptr_t)p % 16) == 0; }

extern "C" int tlc_rmsnorm_add(const float* parts, int n_parts, const float* extra, const float* gate, int gate_ld,
                               int gate_sigmoid, const float* w, float eps, int T, int D, float* res, int accumulate,
                               void* copy, int copy_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(n_parts >= 0 && (n_parts > 0 || extra != nullptr), "rmsnorm_add: nothing to add");
  TLC_REQUIRE(copy == nullptr || copy_dtype == TLC_F32 || copy_dtype == TLC_BF16, "rmsnorm_add: unknown dtype code %d of the copy", copy_dtype);
  if (D % 4 == 0 && D <= 16384 && aligned16(parts) && aligned16(extra) && aligned16(w) && aligned16(res) && aligned16(copy)) {
    const int n4 = D / 4;
#define TLC_RA_LAUNCH(NT, PT)                                                                                             \
  tlc_launch(rmsnorm_add_vec_kernel<NT, PT>, dim3(T), dim3(NT), 0, stream, parts, n_parts, extra, gate, gate_ld, gate_sigmoid, w, \
             eps, D, res, accumulate, copy, copy_dtype)
    if (T >= VEC_MANY_ROWS) { TLC_VEC_SHAPES_MANY(n4, TLC_RA_LAUNCH) } else { TLC_VEC_SHAPES(n4, TLC_RA_LAUNCH) }
#undef TLC_RA_LAUNCH
    TLC_CHECK_LAUNCH("rmsnorm_add");
    return 0;
  }
  const int keep = (size_t)D * sizeof(float) <= 40 * 1024;
  // few rows (single-token steps): more threads a row, so that a thread's loads are few and in flight together
  const int nt = (T < 256 && D >= 1024) ? 1024 : 256;
  tlc_launch(rmsnorm_add_kernel, dim3(T), dim3(nt), keep ? (size_t)D * sizeof(float) : 0, stream, parts, n_parts, extra, gate, gate_ld,
             gate_sigmoid, w, eps, D, res, accumulate, keep, copy, copy_dtype);
  TLC_CHECK_LAUNCH("rmsnorm_add");
  return 0;
}

// ---- gather rows of a 32-bit matrix ------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, int D,
                                   float* __restrict__ out) {
  tlc_pdl(x, rows, out);
  const float* xr = x + (size_t)rows[blockIdx.x] * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[(size_t)blockIdx.x * D + d] = xr[d];
}
extern "C" int tlc_gather_rows(const float* x, const int* rows, int R, int D, float* out, cudaStream_t stream) {
  if (R == 0) return 0;
  tlc_launch(gather_rows_kernel, dim3(R), dim3(256), 0, stream, x, rows, D, out);
  TLC_CHECK_LAUNCH("gather_rows");
  return 0;
}

// ---- a copy of 32-bit rows in the activation type, optionally through tanh ---------------------------------
// Layers whose sublayers read the residual stream itself (no norm in front) take it from here in the type their
// products want; act 1: tanh of every element first (the hidden layer of a small two-layer projection); act 2: the square
// of max(x, 0) (the activation of a feed-forward without a gate).
template <typename TO>
__global__ void convert_kernel(const float* __restrict__ x, int ldx, int D, TO* __restrict__ out, int ldo, size_t total, int act) {
  tlc_pdl(x, out);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / D;
  const int d = (int)(i % D);
  const float v = x[t * ldx + d];
  const float r = fmaxf(v, 0.f);
  out[t * ldo + d] = from_f32<TO>(act == 1 ? tanhf(v) : act == 2 ? r * r : v);
}
// The same, four neighbouring values a thread (widths and strides that are multiples of 4, rows on 16-byte boundaries).
template <typename TO>
__global__ void __launch_bounds__(256)
convert4_kernel(const float* __restrict__ x, int ldx, int D4, TO* __restrict__ out, int ldo, size_t total4, int act) {
  tlc_pdl(x, out);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  const size_t t = i / D4;
  const int d = (int)(i % D4) * 4;
  float4 v = *reinterpret_cast<const float4*>(x + t * ldx + d);
  if (act == 1) { v.x = tanhf(v.x); v.y = tanhf(v.y); v.z = tanhf(v.z); v.w = tanhf(v.w); }
  else if (act == 2) {
    v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
    v.x *= v.x; v.y *= v.y; v.z *= v.z; v.w *= v.w;
  }
  Out4<TO>::put(out + t * ldo + d, v.x, v.y, v.z, v.w);
}
extern "C" int tlc_convert(const float* x, int ldx, int T, int D, void* out, int dtype, int ldo, int act, cudaStream_t stream) {
  const size_t total = (size_t)T * D;
  if (total == 0) return 0;
  if (act >= 0 && act <= 2 && D % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    TLC_DISPATCH_DTYPE(dtype, TO, tlc_launch(convert4_kernel<TO>, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, x, ldx,
                                             D / 4, (TO*)out, ldo, total / 4, act));
    TLC_CHECK_LAUNCH("convert");
    return 0;
  }
  TLC_REQUIRE(act >= 0 && act <= 2, "convert: unknown function %d (0 none, 1 tanh, 2 squared relu)", act);
  TLC_DISPATCH_DTYPE(dtype, TO, tlc_launch(convert_kernel<TO>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, ldx, D,
                                           (TO*)out, ldo, total, act));
  TLC_CHECK_LAUNCH("convert");
  return 0;
}

// ---- x = cap * tanh(x / cap), in place -------------------------------------------------------------------------
__global__ void softcap_kernel(float* x, size_t total, float cap) {
  tlc_pdl(x);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] = cap * tanhf(x[i] / cap);
}
extern "C" int tlc_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  TLC_REQUIRE(cap > 0.f, "softcap: the cap must be positive, got %g", (double)cap);
  tlc_launch(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, (size_t)n, cap);
  TLC_CHECK_LAUNCH("softcap");
  return 0;
}

// ---- the mean of several sublayers' results, each normed by itself ---------------------------------------------------
// y = scale * sum_p parts[t, p, :] / sqrt(mean(parts[t, p, :]^2) + eps) * w[p, :]   (parts [T, n, D], w [n, D]);
// then res[t] (+)= y, or with an outer weight wo: res[t] (+)= y / sqrt(mean(y^2) + eps_o) * wo.  One block per row; all
// statistics 32-bit; y waits in shared memory for its scale where it fits, else it is formed twice.
#define MEAN_MAX_PARTS 8
__global__ void __launch_bounds__(1024)
rmsnorm_mean_add_kernel(const float* __restrict__ parts, int n_parts, const float* __restrict__ w, float eps, float scale,
                        const float* __restrict__ wo, float eps_o, int D, float* __restrict__ res, int accumulate, int keep,
                        void* __restrict__ copy, int copy_dtype) {
  tlc_pdl(parts, res, copy);
  __shared__ float red[33];
  extern __shared__ float yrow[];
  const int t = blockIdx.x;
  const float* pr = parts + (size_t)t * n_parts * D;
  float inv[MEAN_MAX_PARTS];
#pragma unroll
  for (int p = 0; p < MEAN_MAX_PARTS; p++) {
    inv[p] = 0.f;
    if (p < n_parts) {
      float ss = 0.f;
      for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = pr[(size_t)p * D + d]; ss += v * v; }
      ss = block_sum(ss, red);
      inv[p] = scale / sqrtf(ss / (float)D + eps);
    }
  }
  auto mean_at = [&](int d) {
    float y = 0.f;
#pragma unroll
    for (int p = 0; p < MEAN_MAX_PARTS; p++)
      if (p < n_parts) y = fmaf(pr[(size_t)p * D + d] * inv[p], w[(size_t)p * D + d], y);
    return y;
  };
  float s = 1.0f;
  if (wo) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const float y = mean_at(d);
      if (keep) yrow[d] = y;
      ss += y * y;
    }
    ss = block_sum(ss, red);
    s = 1.0f / sqrtf(ss / (float)D + eps_o);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float y = (wo && keep) ? yrow[d] : mean_at(d);          // (yrow[d] was written by this thread)
    const float v = wo ? y * s * wo[d] : y;
    float* o = res + (size_t)t * D + d;
    const float r = accumulate ? *o + v : v;
    *o = r;
    if (copy) put_as(copy, copy_dtype, (size_t)t * D + d, r);
  }
}

// Two summands with both rows in registers: 16-byte loads and stores, the two sums of squares in one pass over the
// block.  D a multiple of 4, at most 4 * NT * PT.
template <int NT, int PT>
__global__ void __launch_bounds__(NT)
rmsnorm_mean2_add_vec_kernel(const float* __restrict__ parts, const float* __restrict__ w, float eps, float scale,
                             const float* __restrict__ wo, float eps_o, int D, float* __restrict__ res, int accumulate,
                             void* __restrict__ copy, int copy_dtype) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[2][33];
  const int n4 = D >> 2, t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float4 w0[PT], w1[PT], a[PT], b[PT];
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    w0[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(w) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    w1[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(w) + n4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tlc_wait(parts, res, copy);
  const float4* pr = reinterpret_cast<const float4*>(parts + (size_t)t * 2 * D);
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    a[i] = c < n4 ? pr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    b[i] = c < n4 ? pr[n4 + c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    sa += a[i].x * a[i].x + a[i].y * a[i].y + a[i].z * a[i].z + a[i].w * a[i].w;
    sb += b[i].x * b[i].x + b[i].y * b[i].y + b[i].z * b[i].z + b[i].w * b[i].w;
  }
  sa = warp_sum(sa);
  sb = warp_sum(sb);
  if (lane == 0) { red[0][warp] = sa; red[1][warp] = sb; }
  __syncthreads();
  if (warp < 2) {
    float x = lane < NT / 32 ? red[warp][lane] : 0.f;
    x = warp_sum(x);
    if (lane == 0) red[warp][32] = x;
  }
  __syncthreads();
  const float ia = scale / sqrtf(red[0][32] / (float)D + eps), ib = scale / sqrtf(red[1][32] / (float)D + eps);
  float4 y[PT], r[PT];
  float4* rr = reinterpret_cast<float4*>(res + (size_t)t * D);
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    r[i] = (accumulate && c < n4) ? rr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    y[i].x = fmaf(b[i].x * ib, w1[i].x, fmaf(a[i].x * ia, w0[i].x, 0.f));
    y[i].y = fmaf(b[i].y * ib, w1[i].y, fmaf(a[i].y * ia, w0[i].y, 0.f));
    y[i].z = fmaf(b[i].z * ib, w1[i].z, fmaf(a[i].z * ia, w0[i].z, 0.f));
    y[i].w = fmaf(b[i].w * ib, w1[i].w, fmaf(a[i].w * ia, w0[i].w, 0.f));
  }
  float s = 1.0f;
  if (wo) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PT; i++) ss += y[i].x * y[i].x + y[i].y * y[i].y + y[i].z * y[i].z + y[i].w * y[i].w;
    ss = block_sum(ss, red[0]);
    s = 1.0f / sqrtf(ss / (float)D + eps_o);
  }
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c >= n4) continue;
    if (wo) {
      const float4 o = __ldg(reinterpret_cast<const float4*>(wo) + c);
      r[i].x += y[i].x * s * o.x; r[i].y += y[i].y * s * o.y; r[i].z += y[i].z * s * o.z; r[i].w += y[i].w * s * o.w;
    } else {
      r[i].x += y[i].x; r[i].y += y[i].y; r[i].z += y[i].z; r[i].w += y[i].w;
    }
    rr[c] = r[i];
    if (copy) put4_as(copy, copy_dtype, (size_t)t * D + 4 * c, r[i]);
  }
}
extern "C" int tlc_rmsnorm_mean_add(const float* parts, int n_parts, const float* w, float eps, float scale, const float* wo,
                                    float eps_o, int T, int D, float* res, int accumulate, void* copy, int copy_dtype,
                                    cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(n_parts >= 1 && n_parts <= MEAN_MAX_PARTS, "rmsnorm_mean_add: %d summands (1..%d)", n_parts, MEAN_MAX_PARTS);
  TLC_REQUIRE(copy == nullptr || copy_dtype == TLC_F32 || copy_dtype == TLC_BF16, "rmsnorm_mean_add: unknown dtype code %d of the copy", copy_dtype);
  if (n_parts == 2 && D % 4 == 0 && D <= 16384 && aligned16(parts) && aligned16(w) && aligned16(wo) && aligned16(res) && aligned16(copy)) {
    const int n4 = D / 4;
#define TLC_RM_LAUNCH(NT, PT)                                                                                           \
  tlc_launch(rmsnorm_mean2_add_vec_kernel<NT, PT>, dim3(T), dim3(NT), 0, stream, parts, w, eps, scale, wo, eps_o, D, res, accumulate, \
             copy, copy_dtype)
    if (T >= VEC_MANY_ROWS) { TLC_VEC_SHAPES_MANY(n4, TLC_RM_LAUNCH) } else { TLC_VEC_SHAPES(n4, TLC_RM_LAUNCH) }
#undef TLC_RM_LAUNCH
    TLC_CHECK_LAUNCH("rmsnorm_mean_add");
    return 0;
  }
  const int keep = (size_t)D * sizeof(float) <= 40 * 1024;
  const int nt = (T < 256 && D >= 1024) ? 1024 : 256;
  tlc_launch(rmsnorm_mean_add_kernel, dim3(T), dim3(nt), keep ? (size_t)D * sizeof(float) : 0, stream, parts, n_parts, w, eps, scale, wo,
             eps_o, D, res, accumulate, keep, copy, copy_dtype);
  TLC_CHECK_LAUNCH("rmsnorm_mean_add");
  return 0;
}
