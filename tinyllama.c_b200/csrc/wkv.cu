// A time-mixing layer with a decaying matrix state per head and a bonus for the current token:
//
//   o_t = (S + diag(u) k_t v_t^T)^T r_t          S <- diag(w_t) S + k_t v_t^T          w_t = exp(-exp(a_t))
//
// S [d, d] per head (rows: key channels, columns: value channels), 32-bit, carried per sequence; u [H, d] learned; r, k, v
// and the decay's logarithm a arrive as columns of 32-bit projections.  Every projection of such a layer reads a mix of
// its own of the token's input and the previous token's: m_s[t] = x[t] + (x[t-1] - x[t]) * mu_s (tlc_shift_mix), the
// previous token's row being part of the sequence's state as well.
//
// The scan (tlc_wkv_scan): column j of S depends on column j alone.  A block owns a group of columns of one (sequence,
// head); a column's rows are split among R neighbouring lanes (R a power of two up to 32), each lane holding NC chunks of
// four rows in registers (chunk c of lane p: rows 4 (c R + p) ..., so that the lanes of a column read r, k and w of a
// token as neighbouring 16-byte words of shared memory), and the lanes join their partial read-outs by shuffles.  The
// bonus term is the same for every column, v_j * sum_i r_i u_i k_i: that sum is taken once per token.  Tokens arrive in
// tiles of 16 by cp.async, the next tile while the current one is walked; a pass over the tile takes the decay's two
// exponentials once per element; a tile's outputs leave through shared memory in whole rows.  The state is read once and
// written once per step.
#include "common.cuh"

#define WKV_TOK 16           // tokens a tile
#define WKV_THREADS 256      // threads a block at most

// out[t, s, :] = x[t] + (prev - x[t]) * mu[s], prev the row above or the slot's kept row (zeros at position 0); the block of
// a sequence's first row of the step, the only one that reads the slot, afterwards leaves the sequence's last row there.
template <typename TO>
__global__ void __launch_bounds__(256)
shift_mix_kernel(const float* __restrict__ x, const float* __restrict__ mu, int n_mix, int D, const int* __restrict__ row_seq,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots, const int* __restrict__ start_pos, float* state,
                 TO* __restrict__ out) {
  tlc_pdl(x, state, out);
  const int t = blockIdx.x, b = row_seq[t];
  const int first = cu_seqlens[b], last = cu_seqlens[b + 1] - 1;
  const float* xr = x + (size_t)t * D;
  float* st = state + (size_t)slots[b] * D;
  const bool from_state = t == first, fresh = start_pos[b] == 0;
  const float* xl = x + (size_t)last * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float cur = xr[d];
    const float prev = from_state ? (fresh ? 0.f : st[d]) : xr[d - D];
    const float diff = prev - cur;
    for (int s = 0; s < n_mix; s++)
      out[((size_t)t * n_mix + s) * D + d] = from_f32<TO>(fmaf(diff, mu[(size_t)s * D + d], cur));
    if (from_state) st[d] = xl[d];           // (read above by this thread)
  }
}

extern "C" int tlc_shift_mix(const float* x, const float* mu, int n_mix, int T, int D, const int* row_seq, const int* cu_seqlens,
                             const int* slots, const int* start_pos, float* state, void* out, int out_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(n_mix >= 1, "shift_mix: %d mixes", n_mix);
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(shift_mix_kernel<TO>, dim3(T), dim3(256), 0, stream, x, mu, n_mix, D, row_seq, cu_seqlens,
                                               slots, start_pos, state, (TO*)out));
  TLC_CHECK_LAUNCH("shift_mix");
  return 0;
}

__device__ __forceinline__ void wkv_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void wkv_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void wkv_cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int R, int NC>
__global__ void __launch_bounds__(WKV_THREADS)
wkv_scan_kernel(const float* __restrict__ rkv, int ld, int r_off, int k_off, int v_off, const float* __restrict__ decay_log, int ld_w,
                const float* __restrict__ bonus, float* state, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                const int* __restrict__ start_pos, int H, int d, int COLS, float* __restrict__ out, int out_ld) {
  tlc_pdl(rkv, decay_log, state, out);
  constexpr int DP = 4 * R * NC;              // rows of a column, padded (rows from d on stay zero)
  constexpr int CPW = 32 / R;                 // columns a warp
  extern __shared__ __align__(16) float wkv_sh[];
  const int tile_floats = 3 * WKV_TOK * DP + WKV_TOK * COLS;     // r | k | a, then w | v
  float* es = wkv_sh + 2 * tile_floats;       // [WKV_TOK]: sum_i r_i u_i k_i of the tile's tokens
  float* os = es + WKV_TOK;                   // [WKV_TOK][COLS]: the tile's outputs
  float* us = os + WKV_TOK * COLS;            // [DP]
  const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * COLS;
  const int tid = threadIdx.x, nt = blockDim.x, warp = tid >> 5, lane = tid & 31, n_warps = nt >> 5;
  const int part = lane % R, jj = warp * CPW + lane / R, j = j0 + jj;
  const bool col = j < d;
  float S[NC][4];
  float* sp = state + (((size_t)slots[b] * H + h) * d) * d;
  const bool fresh = start_pos[b] == 0;
#pragma unroll
  for (int c = 0; c < NC; c++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int row = (c * R + part) * 4 + e;
      S[c][e] = (!fresh && col && row < d) ? sp[(size_t)row * d + j] : 0.f;
    }
  for (int i = tid; i < DP; i += nt) us[i] = i < d ? bonus[(size_t)h * d + i] : 0.f;
  for (int bufi = 0; bufi < 2; bufi++)        // the padded rows, which no copy writes
    for (int idx = tid; idx < 3 * WKV_TOK * (DP - d); idx += nt) {
      const int a = idx / (DP - d), i = d + idx % (DP - d);
      wkv_sh[bufi * tile_floats + a * DP + i] = 0.f;
    }
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const size_t head = (size_t)h * d;
  // element e of a tile's [n, d] (or [n, COLS]) arrays, e = tid, tid + nt, ...: its token and channel advance without a division
  const int d_tt = nt / d, d_i = nt % d, c_tt = nt / COLS, c_i = nt % COLS;
  auto fetch = [&](int tb, int bufi) {
    const int n = min(WKV_TOK, t1 - tb);
    float* rs = wkv_sh + bufi * tile_floats;
    float *ks = rs + WKV_TOK * DP, *as = ks + WKV_TOK * DP, *vs = as + WKV_TOK * DP;
    for (int tt = tid / d, i = tid % d; tt < n; tt += d_tt, i += d_i) {
      if (i >= d) { i -= d; tt++; if (tt >= n) break; }
      const float* pr = rkv + (size_t)(tb + tt) * ld + head + i;
      wkv_cp4(rs + tt * DP + i, pr + r_off);
      wkv_cp4(ks + tt * DP + i, pr + k_off);
      wkv_cp4(as + tt * DP + i, decay_log + (size_t)(tb + tt) * ld_w + head + i);
    }
    for (int tt = tid / COLS, c = tid % COLS; tt < n; tt += c_tt, c += c_i) {
      if (c >= COLS) { c -= COLS; tt++; if (tt >= n) break; }
      if (j0 + c < d) wkv_cp4(vs + tt * COLS + c, rkv + (size_t)(tb + tt) * ld + v_off + head + j0 + c);
      else vs[tt * COLS + c] = 0.f;
    }
    wkv_cp_commit();
  };
  if (t0 < t1) fetch(t0, 0);
  int bufi = 0;
  for (int tb = t0; tb < t1; tb += WKV_TOK, bufi ^= 1) {
    const int n = min(WKV_TOK, t1 - tb);
    wkv_cp_wait_all();
    __syncthreads();                          // this tile has landed; the tile before is walked and its outputs are out
    if (tb + WKV_TOK < t1) fetch(tb + WKV_TOK, bufi ^ 1);
    float* rs = wkv_sh + bufi * tile_floats;
    float *ks = rs + WKV_TOK * DP, *ws = ks + WKV_TOK * DP, *vs = ws + WKV_TOK * DP;
    for (int tt = tid / d, i = tid % d; tt < n; tt += d_tt, i += d_i) {
      if (i >= d) { i -= d; tt++; if (tt >= n) break; }
      ws[tt * DP + i] = expf(-expf(ws[tt * DP + i]));
    }
    for (int tt = warp; tt < n; tt += n_warps) {
      float e = 0.f;
      for (int i = lane; i < d; i += 32) e = fmaf(rs[tt * DP + i] * us[i], ks[tt * DP + i], e);
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) e += __shfl_xor_sync(0xffffffffu, e, s);
      if (lane == 0) es[tt] = e;
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < n; tt++) {
      const float4* r4 = reinterpret_cast<const float4*>(rs + tt * DP);
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DP);
      const float4* w4 = reinterpret_cast<const float4*>(ws + tt * DP);
      const float v = vs[tt * COLS + jj];
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int c = 0; c < NC; c++) {
        const float4 r = r4[c * R + part], k = k4[c * R + part], w = w4[c * R + part];
        o0 = fmaf(r.x, S[c][0], o0);
        o1 = fmaf(r.y, S[c][1], o1);
        o0 = fmaf(r.z, S[c][2], o0);
        o1 = fmaf(r.w, S[c][3], o1);
        S[c][0] = fmaf(w.x, S[c][0], k.x * v);
        S[c][1] = fmaf(w.y, S[c][1], k.y * v);
        S[c][2] = fmaf(w.z, S[c][2], k.z * v);
        S[c][3] = fmaf(w.w, S[c][3], k.w * v);
      }
      float o = o0 + o1;
#pragma unroll
      for (int s = 1; s < R; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
      if (part == 0) os[tt * COLS + jj] = fmaf(es[tt], v, o);
    }
    __syncthreads();
    for (int tt = tid / COLS, c = tid % COLS; tt < n; tt += c_tt, c += c_i) {
      if (c >= COLS) { c -= COLS; tt++; if (tt >= n) break; }
      if (j0 + c < d) out[(size_t)(tb + tt) * out_ld + head + j0 + c] = os[tt * COLS + c];
    }
  }
#pragma unroll
  for (int c = 0; c < NC; c++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int row = (c * R + part) * 4 + e;
      if (col && row < d) sp[(size_t)row * d + j] = S[c][e];
    }
}

template <int R, int NC>
static void wkv_launch(dim3 grid, int threads, size_t smem, cudaStream_t stream, const float* rkv, int ld, int r_off, int k_off,
                       int v_off, const float* decay_log, int ld_w, const float* bonus, float* state, const int* cu_seqlens,
                       const int* slots, const int* start_pos, int H, int d, int COLS, float* out, int out_ld) {
  // (more than 48 KB of dynamic shared memory, which the widest heads need, must be asked for)
  if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<R, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  tlc_launch(wkv_scan_kernel<R, NC>, grid, dim3(threads), smem, stream, rkv, ld, r_off, k_off, v_off, decay_log, ld_w, bonus, state,
             cu_seqlens, slots, start_pos, H, d, COLS, out, out_ld);
}

extern "C" int tlc_wkv_scan(const float* rkv, int ld, int r_off, int k_off, int v_off, const float* decay_log, int ld_w,
                            const float* bonus, float* state, const int* cu_seqlens, const int* slots, const int* start_pos, int B,
                            int H, int d, float* out, int out_ld, cudaStream_t stream) {
  if (B == 0 || H == 0) return 0;
  TLC_REQUIRE(d >= 1 && d <= 256, "wkv_scan: heads of %d channels are outside what the kernel is built for (1..256)", d);
  TLC_REQUIRE(H <= 65535, "wkv_scan: too many heads (%d)", H);
  // lanes a column and chunks of four rows a lane: eight rows a lane, or twelve on half the lanes where those hold the head
  int R = 1, NC = d <= 4 ? 1 : 2;
  while (R * 8 < d) R <<= 1;
  if (R >= 2 && (R / 2) * 12 >= d) { R /= 2; NC = 3; }
  const int cpw = 32 / R, DP = 4 * R * NC;
  const int COLS = min(WKV_THREADS / R, (d + cpw - 1) / cpw * cpw);
  const size_t smem = ((size_t)2 * (3 * WKV_TOK * DP + WKV_TOK * COLS) + WKV_TOK + (size_t)WKV_TOK * COLS + DP) * sizeof(float);
  dim3 grid(B, H, (d + COLS - 1) / COLS);
#define WKV_CASE(RR, CC)                                                                                                       \
  if (R == RR && NC == CC) {                                                                                                    \
    wkv_launch<RR, CC>(grid, COLS * R, smem, stream, rkv, ld, r_off, k_off, v_off, decay_log, ld_w, bonus, state, cu_seqlens,     \
                       slots, start_pos, H, d, COLS, out, out_ld);                                                              \
  } else
  WKV_CASE(1, 1) WKV_CASE(1, 2) WKV_CASE(2, 2) WKV_CASE(4, 2) WKV_CASE(8, 2) WKV_CASE(16, 2) WKV_CASE(32, 2)
  WKV_CASE(1, 3) WKV_CASE(2, 3) WKV_CASE(4, 3) WKV_CASE(8, 3) WKV_CASE(16, 3)
  TLC_REQUIRE(false, "wkv_scan: no kernel for %d lanes a column with %d chunks", R, NC);
#undef WKV_CASE
  TLC_CHECK_LAUNCH("wkv_scan");
  return 0;
}
