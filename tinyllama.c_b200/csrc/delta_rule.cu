// The gated delta rule: a recurrence over tokens whose state is a matrix per head, corrected towards every new
// (key, value) pair instead of merely summing them.
//
// Per head, with the token's unit-length key k and query q (dk values), value v (dv values), write strength b in (0, 1)
// and decay a in (0, 1], and the state M [dk, dv] (32-bit, zero at position 0, kept per sequence between steps): the state
// is decayed, asked what it would return for the new key (the prediction p), corrected by the write w, and read:
//   M <- a M;   p = M^T k;   w = b (v - p);   M <- M + k w^T;   r = M^T q
// (the read-out comes last: it already contains what this token wrote; in the code M is S, w is u, a is g, b is bt).
// Several value heads may share a query/key head (value head i reads query/key head i / (H / G)).
//
// Column j of M depends on column j alone: w_j = b (v_j - M[:, j] . k), M[:, j] <- a M[:, j] + k w_j, r_j = M[:, j] . q.
// So a group of NS threads (neighbouring lanes) owns four columns: each holds DKQ rows of them in registers; the group
// walks the sequence's rows of this step in order and joins its partial dot products by shuffles.  A block takes 32
// columns of one (sequence, head).  Everything is 32-bit.
//
// tlc_delta_prepare makes the inputs of the walk, a warp per (row, query or key head), in place in the 32-bit buffer that
// holds q | k | v after the short convolution: x / sqrt(sum(x^2) + l2_eps), the query also times q_scale; and
// beta = sigmoid of the row's write-strength projection, one per head.
#include "common.cuh"

__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ qkv, int ld, int q_off, int k_off, int G, int dk, float l2_eps, float q_scale,
                     const float* __restrict__ proj, int ldp, int b_off, int H, float* __restrict__ beta, int T,
                     float* __restrict__ chan, int ldc, const float* __restrict__ A) {
  tlc_pdl(qkv, proj, beta, chan);
  const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int units = 2 * G + (chan ? H : 0);
  if (w >= T * units) return;
  const int t = w / units, u = w - t * units;
  if (u >= 2 * G) {       // a decay per key channel of head h, in place: exp(A[h] * softplus(x)), A[h] = -exp(A_log[h])
    const int h = u - 2 * G;
    float* c = chan + (size_t)t * ldc + (size_t)h * dk;
    const float a = A[h];
    for (int d = lane; d < dk; d += 32) {
      const float x = c[d];
      const float sp = x > 20.f ? x : log1pf(expf(x));
      c[d] = expf(a * sp);
    }
    return;
  }
  if (u == 0)
    for (int h = lane; h < H; h += 32) beta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-proj[(size_t)t * ldp + b_off + h]));
  float* x = qkv + (size_t)t * ld + (u < G ? q_off + u * dk : k_off + (u - G) * dk);
  float ss = 0.f;
  for (int d = lane; d < dk; d += 32) { const float v = x[d]; ss += v * v; }
  ss = warp_sum(ss);
  const float s = (u < G ? q_scale : 1.0f) / sqrtf(ss + l2_eps);
  for (int d = lane; d < dk; d += 32) x[d] *= s;
}

extern "C" int tlc_delta_prepare(float* qkv, int ld, int q_off, int k_off, int G, int dk, float l2_eps, float q_scale,
                                 const float* proj, int ldp, int b_off, int H, float* beta, int T, float* chan, int ldc,
                                 const float* A, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(G >= 1 && dk >= 1 && H >= 1, "delta_prepare: bad sizes G=%d dk=%d H=%d", G, dk, H);
  TLC_REQUIRE(chan == nullptr || (A != nullptr && ldc >= H * dk), "delta_prepare: decays per channel need A [H] and rows of H * dk values");
  const long long warps = (long long)T * (2 * G + (chan ? H : 0));
  tlc_launch(delta_prepare_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, qkv, ld, q_off, k_off, G, dk, l2_eps, q_scale,
             proj, ldp, b_off, H, beta, T, chan, ldc, A);
  TLC_CHECK_LAUNCH("delta_prepare");
  return 0;
}

#define DELTA_COLS 32     // columns of S a block takes
#define DELTA_CT 4        // columns of S a thread takes

__device__ __forceinline__ void delta_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void delta_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
template <int N> __device__ __forceinline__ void delta_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Thread (cg, s), s the fastest index: columns j0 + 4 cg .. + 3, rows s * DKQ .. s * DKQ + DKQ - 1 of S: a tile of
// DKQ x 4 elements in registers, so that a value of k or q fetched from shared memory serves four multiply-adds (with one
// column a thread the kernel was bound by its shared-memory instructions: a token took 800 cycles).  The NS threads of
// a column group join their partial dot products by shuffles.  The tokens' keys, queries, values, decays and write
// strengths arrive in tiles of TT tokens by cp.async, the next tile while the current one is walked.  In shared memory a
// token's key is laid out thread by thread, DKQ values and DKS - DKQ of padding each, so that the 16-byte pieces the
// lanes of a quarter warp read lie in different banks.
// CH: the decay is a vector per token and head, one factor per ROW of S (key channel): decay [T, ldd], head h at column
// h * dk; it travels with the key, laid out like it.  (a M)^T k is then no multiple of M^T k: the rows are decayed first.
template <int DKQ, int NS, int TT, bool CH>
__global__ void __launch_bounds__(DELTA_COLS / DELTA_CT * NS)
delta_rule_kernel(const float* __restrict__ qkv, int ld, int q_off, int k_off, int v_off, const float* __restrict__ beta,
                  const float* __restrict__ decay, float* state, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ slots, const int* __restrict__ start_pos, int H, int G, int dk, int dv,
                  float* __restrict__ y, int ldy, int vec, int ldd) {
  tlc_pdl(qkv, beta, decay, state, y);
  constexpr int CT = DELTA_CT, NT = DELTA_COLS / CT * NS, DKS = DKQ == 4 ? 4 : DKQ + 4, KROW = NS * DKS;
  constexpr int NKQ = CH ? 3 : 2;                                   // vectors of dk values a token brings: k, q (and the decays)
  constexpr int STAGE = TT * (NKQ * KROW + DELTA_COLS + 4);         // floats: k, q (, decays) [TT][KROW]; v [TT][32]; decay, beta [TT][2] (+2)
  __shared__ __align__(16) float sm[2 * STAGE];
  const int b = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
  const int cg = tid / NS, s = tid % NS;
  const int j0 = blockIdx.x * DELTA_COLS, jc = j0 + cg * CT;        // this thread's first column
  const int kvh = h / (H / G);
  float* st = state + (((size_t)slots[b] * H + h) * dk) * dv;
  float S[DKQ][CT];
  const bool fresh = start_pos[b] == 0;
#pragma unroll
  for (int i = 0; i < DKQ; i++) {
    const int r = s * DKQ + i;
#pragma unroll
    for (int cc = 0; cc < CT; cc++) S[i][cc] = (!fresh && r < dk && jc + cc < dv) ? st[(size_t)r * dv + jc + cc] : 0.f;
  }
  if (dk != DKQ * NS || dv - j0 < DELTA_COLS || DKS != DKQ)          // rows past dk, columns past dv and padding stay zero
    for (int i = tid; i < 2 * STAGE; i += NT) sm[i] = 0.f;
  __syncthreads();
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const int n_tiles = (t1 - t0 + TT - 1) / TT;
  const int n_cols = min(DELTA_COLS, dv - j0);
  auto load = [&](int tile, int buf) {
    float* base = sm + buf * STAGE;
    const int ta = t0 + tile * TT, nt = min(TT, t1 - ta);
    if (vec) {                                          // 16-byte copies (4-byte ones are several times slower a byte)
      const int dk4 = dk >> 2, nc4 = n_cols >> 2;
      for (int i = tid; i < nt * dk4; i += NT) {
        const int tt = i / dk4, r = (i - tt * dk4) << 2;
        const int at = tt * KROW + (r / DKQ) * DKS + (r % DKQ);
        const float* row = qkv + (size_t)(ta + tt) * ld;
        delta_cp16(base + at, row + k_off + kvh * dk + r);
        delta_cp16(base + TT * KROW + at, row + q_off + kvh * dk + r);
        if (CH) delta_cp16(base + 2 * TT * KROW + at, decay + (size_t)(ta + tt) * ldd + h * dk + r);
      }
      for (int i = tid; i < nt * nc4; i += NT) {
        const int tt = i / nc4, cc = (i - tt * nc4) << 2;
        delta_cp16(base + NKQ * TT * KROW + tt * DELTA_COLS + cc, qkv + (size_t)(ta + tt) * ld + v_off + h * dv + j0 + cc);
      }
    } else {
      for (int i = tid; i < nt * dk; i += NT) {
        const int tt = i / dk, r = i - tt * dk;
        const int at = tt * KROW + (r / DKQ) * DKS + (r % DKQ);
        const float* row = qkv + (size_t)(ta + tt) * ld;
        delta_cp4(base + at, row + k_off + kvh * dk + r);
        delta_cp4(base + TT * KROW + at, row + q_off + kvh * dk + r);
        if (CH) delta_cp4(base + 2 * TT * KROW + at, decay + (size_t)(ta + tt) * ldd + h * dk + r);
      }
      for (int i = tid; i < nt * n_cols; i += NT) {
        const int tt = i / n_cols, cc = i - tt * n_cols;
        delta_cp4(base + NKQ * TT * KROW + tt * DELTA_COLS + cc, qkv + (size_t)(ta + tt) * ld + v_off + h * dv + j0 + cc);
      }
    }
    if (tid < nt) {
      if (!CH) delta_cp4(base + NKQ * TT * KROW + TT * DELTA_COLS + 2 * tid, decay + (size_t)(ta + tid) * H + h);
      delta_cp4(base + NKQ * TT * KROW + TT * DELTA_COLS + 2 * tid + 1, beta + (size_t)(ta + tid) * H + h);
    }
  };
  if (n_tiles > 0) load(0, 0);
  delta_cp_commit();
  for (int tile = 0; tile < n_tiles; tile++) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) load(tile + 1, buf ^ 1);
    delta_cp_commit();
    delta_cp_wait<1>();
    __syncthreads();
    const float* ks = sm + buf * STAGE + s * DKS;       // this thread's rows of every key
    const float* qs = ks + TT * KROW;
    const float* gs = qs + TT * KROW;                   // (CH) this thread's rows of every token's decays
    const float* vs = sm + buf * STAGE + NKQ * TT * KROW + cg * CT;
    const float* gb = sm + buf * STAGE + NKQ * TT * KROW + TT * DELTA_COLS;
    const int ta = t0 + tile * TT, nt = min(TT, t1 - ta);
    for (int tt = 0; tt < nt; tt++) {
      float kk[DKQ], qq[DKQ];
#pragma unroll
      for (int i = 0; i < DKQ; i += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(ks + tt * KROW + i);
        const float4 qv = *reinterpret_cast<const float4*>(qs + tt * KROW + i);
        kk[i] = kv.x; kk[i + 1] = kv.y; kk[i + 2] = kv.z; kk[i + 3] = kv.w;
        qq[i] = qv.x; qq[i + 1] = qv.y; qq[i + 2] = qv.z; qq[i + 3] = qv.w;
      }
      const float4 vv = *reinterpret_cast<const float4*>(vs + tt * DELTA_COLS);
      const float2 gbt = *reinterpret_cast<const float2*>(gb + 2 * tt);
      const float g = CH ? 1.0f : gbt.x, bt = gbt.y;
      float d[CT];
#pragma unroll
      for (int cc = 0; cc < CT; cc++) d[cc] = 0.f;
      if (CH) {                                         // every row by its own factor, before the state is asked
#pragma unroll
        for (int i = 0; i < DKQ; i += 4) {
          const float4 gv = *reinterpret_cast<const float4*>(gs + tt * KROW + i);
          const float gg[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
          for (int e = 0; e < 4; e++)
#pragma unroll
            for (int cc = 0; cc < CT; cc++) S[i + e][cc] *= gg[e];
        }
      }
#pragma unroll
      for (int i = 0; i < DKQ; i++)
#pragma unroll
        for (int cc = 0; cc < CT; cc++) d[cc] = fmaf(S[i][cc], kk[i], d[cc]);
#pragma unroll
      for (int o = 1; o < NS; o <<= 1)
#pragma unroll
        for (int cc = 0; cc < CT; cc++) d[cc] += __shfl_xor_sync(0xffffffffu, d[cc], o);
      float u[CT];                                      // the decayed state's prediction: (a M)^T k = a (M^T k)
      u[0] = bt * (vv.x - g * d[0]); u[1] = bt * (vv.y - g * d[1]); u[2] = bt * (vv.z - g * d[2]); u[3] = bt * (vv.w - g * d[3]);
      float out[CT];
#pragma unroll
      for (int cc = 0; cc < CT; cc++) out[cc] = 0.f;
#pragma unroll
      for (int i = 0; i < DKQ; i++)
#pragma unroll
        for (int cc = 0; cc < CT; cc++) {
          S[i][cc] = fmaf(kk[i], u[cc], CH ? S[i][cc] : g * S[i][cc]);
          out[cc] = fmaf(S[i][cc], qq[i], out[cc]);
        }
#pragma unroll
      for (int o = 1; o < NS; o <<= 1)
#pragma unroll
        for (int cc = 0; cc < CT; cc++) out[cc] += __shfl_xor_sync(0xffffffffu, out[cc], o);
      if (s == 0) {
        float* yo = y + (size_t)(ta + tt) * ldy + h * dv + jc;
#pragma unroll
        for (int cc = 0; cc < CT; cc++)
          if (jc + cc < dv) yo[cc] = out[cc];
      }
    }
    __syncthreads();                                    // the tile's buffer is free for the tile after the next
  }
  delta_cp_wait<0>();
#pragma unroll
  for (int i = 0; i < DKQ; i++) {
    const int r = s * DKQ + i;
#pragma unroll
    for (int cc = 0; cc < CT; cc++)
      if (r < dk && jc + cc < dv) st[(size_t)r * dv + jc + cc] = S[i][cc];
  }
}

static int g_delta_split = 0;
// Fixes how many threads share the rows of a column group of the state (8 or 16; 0: chosen); for tests and comparisons.
extern "C" void tlc_delta_rule_split(int threads) { g_delta_split = (threads == 8 || threads == 16) ? threads : 0; }

// qkv float [T, ld]: the normalised queries (G heads of dk) at q_off, keys at k_off, values (H heads of dv) at v_off;
// beta, decay float [T, H]; state float [n_slots, H, dk, dv], updated in place (a sequence at position 0 starts from
// zero whatever its slot holds); y float [T, ldy] receives the read-outs, head h at column h * dv.  B sequences, T rows in all.
extern "C" int tlc_delta_rule(const float* qkv, int ld, int q_off, int k_off, int v_off, const float* beta, const float* decay,
                              float* state, const int* cu_seqlens, const int* slots, const int* start_pos, int B, int T, int H,
                              int G, int dk, int dv, float* y, int ldy, int ldd, cudaStream_t stream) {
  if (B == 0) return 0;
  TLC_REQUIRE(H >= 1 && G >= 1 && H % G == 0 && H <= 65535 && B <= 65535, "delta_rule: %d heads over %d query/key heads, %d sequences", H, G, B);
  TLC_REQUIRE(dk >= 1 && dk <= 256 && dv >= 1, "delta_rule: keys of %d values exceed the kernel's limit of 256", dk);
  const dim3 grid((dv + DELTA_COLS - 1) / DELTA_COLS, H, B);
  // whether every piece of four keys, queries or values starts on a 16-byte boundary
  const int vec = ((uintptr_t)qkv % 16 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 && dk % 4 == 0 &&
                   dv % 4 == 0 && (ldd == 0 || ((uintptr_t)decay % 16 == 0 && ldd % 4 == 0))) ? 1 : 0;
  TLC_REQUIRE(ldd == 0 || ldd >= H * dk, "delta_rule: decays per channel in rows of %d values for %d heads of %d", ldd, H, dk);
#define DELTA_LAUNCH_AS(DKQ, NS, TT, CH)                                                                                    \
  tlc_launch(delta_rule_kernel<DKQ, NS, TT, CH>, grid, dim3(DELTA_COLS / DELTA_CT * NS), 0, stream, qkv, ld, q_off, k_off, v_off, beta, \
             decay, state, cu_seqlens, slots, start_pos, H, G, dk, dv, y, ldy, vec, ldd)
  // (with a decay per channel a token brings three vectors of dk values: half the tokens a tile where two tiles of
  // the larger shapes would not fit the 48 KB of static shared memory)
#define DELTA_LAUNCH(DKQ, NS, TT)                                                                                           \
  do { if (ldd > 0) { DELTA_LAUNCH_AS(DKQ, NS, (TT * (3 * NS * (DKQ == 4 ? 4 : DKQ + 4) + DELTA_COLS + 4) * 8 > 48 * 1024 ? TT / 2 : TT), true); } \
       else { DELTA_LAUNCH_AS(DKQ, NS, TT, false); } } while (0)
  // threads that share the rows of a column group, unless told otherwise: sixteen with few rows each for prompts, eight
  // with twice the rows for single-token steps (T == B), which move the state once and are bound by that traffic
  // (16 heads of 128 x 128: a 2,048-token prompt 755 against 876 us, 64 single tokens 54 against 34 us)
  const int ns = g_delta_split ? g_delta_split : (T > B ? 16 : 8);
  if (dk <= 32) DELTA_LAUNCH(4, 8, 16);
  else if (dk <= 64) { if (ns == 16) DELTA_LAUNCH(4, 16, 16); else DELTA_LAUNCH(8, 8, 16); }
  else if (dk <= 128) { if (ns == 16) DELTA_LAUNCH(8, 16, 8); else DELTA_LAUNCH(16, 8, 16); }
  else DELTA_LAUNCH(16, 16, 8);
#undef DELTA_LAUNCH
#undef DELTA_LAUNCH_AS
  TLC_CHECK_LAUNCH("delta_rule");
  return 0;
}
