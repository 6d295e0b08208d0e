// The gated delta rule: a recurrence over tokens whose state is a matrix per head, corrected towards every new
// (key, value) pair instead of merely summing them.
//
// Per head, with the token's unit-length key k and query q (dk values), value v (dv values), write strength beta in (0, 1)
// and decay g in (0, 1], and the state S [dk, dv] (32-bit, zero at position 0, kept per sequence between steps):
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// in this order, so the read-out sees the token's own write.  Query and key heads may be shared by several value heads
// (head h uses q/k head h / (H / G)).
//
// Column j of S depends on column j alone: u_j = beta (v_j - S[:, j] . k), S[:, j] <- g S[:, j] + k u_j, o_j = S[:, j] . q.
// So a thread group owns a column: NS threads (neighbouring lanes) hold DKQ rows each of it in registers, walk the
// sequence's rows of this step in order and join their partial dot products by shuffles.  A block takes 32 columns of
// one (sequence, head).  Everything is 32-bit.
//
// tlc_delta_prepare makes the inputs of the walk, a warp per (row, query or key head), in place in the 32-bit buffer that
// holds q | k | v after the short convolution: x / sqrt(sum(x^2) + l2_eps), the query also times q_scale; and
// beta = sigmoid of the row's write-strength projection, one per head.
#include "common.cuh"

__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ qkv, int ld, int q_off, int k_off, int G, int dk, float l2_eps, float q_scale,
                     const float* __restrict__ proj, int ldp, int b_off, int H, float* __restrict__ beta, int T) {
  tlc_pdl(qkv, proj, beta);
  const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int units = 2 * G;
  if (w >= T * units) return;
  const int t = w / units, u = w - t * units;
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
                                 const float* proj, int ldp, int b_off, int H, float* beta, int T, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(G >= 1 && dk >= 1 && H >= 1, "delta_prepare: bad sizes G=%d dk=%d H=%d", G, dk, H);
  const long long warps = (long long)T * 2 * G;
  tlc_launch(delta_prepare_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, qkv, ld, q_off, k_off, G, dk, l2_eps, q_scale,
             proj, ldp, b_off, H, beta, T);
  TLC_CHECK_LAUNCH("delta_prepare");
  return 0;
}

#define DELTA_COLS 32     // columns of S a block takes

__device__ __forceinline__ void delta_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void delta_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Thread (c, s), s the fastest index: column j0 + c, rows s, s + NS, s + 2 NS, ... of S.  The tokens' keys, queries,
// values, decays and write strengths arrive in tiles of TT tokens by cp.async, the next tile while the current one
// is walked: a token's step is then arithmetic and two rounds of shuffles, with no trip to memory on its path.
// TT: tokens of a tile that is staged in shared memory (two tiles: one in use, one on its way).
template <int DKQ, int NS, int TT>
__global__ void __launch_bounds__(DELTA_COLS * NS)
delta_rule_kernel(const float* __restrict__ qkv, int ld, int q_off, int k_off, int v_off, const float* __restrict__ beta,
                  const float* __restrict__ decay, float* state, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ slots, const int* __restrict__ start_pos, int H, int G, int dk, int dv,
                  float* __restrict__ y, int ldy) {
  tlc_pdl(qkv, beta, decay, state, y);
  constexpr int NT = DELTA_COLS * NS, DKP = DKQ * NS;
  constexpr int STAGE = TT * (2 * DKP + DELTA_COLS + 2);       // floats: k, q [TT][DKP]; v [TT][32]; decay, beta [TT]
  __shared__ float sm[2 * STAGE];
  const int b = blockIdx.z, h = blockIdx.y, tid = threadIdx.x;
  const int c = tid / NS, s = tid % NS;
  const int j0 = blockIdx.x * DELTA_COLS, j = j0 + c;
  const bool col_ok = j < dv;
  const int kvh = h / (H / G);
  float* st = state + (((size_t)slots[b] * H + h) * dk) * dv + (col_ok ? j : 0);
  float S[DKQ];
  const bool fresh = start_pos[b] == 0;
#pragma unroll
  for (int i = 0; i < DKQ; i++) {
    const int r = s + i * NS;
    S[i] = (!fresh && col_ok && r < dk) ? st[(size_t)r * dv] : 0.f;
  }
  if (dk != DKP || dv - j0 < DELTA_COLS)                             // rows past dk and columns past dv stay zero
    for (int i = tid; i < 2 * STAGE; i += NT) sm[i] = 0.f;
  __syncthreads();
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const int n_tiles = (t1 - t0 + TT - 1) / TT;
  const int n_cols = min(DELTA_COLS, dv - j0);
  auto load = [&](int tile, int buf) {
    float* base = sm + buf * STAGE;
    const int ta = t0 + tile * TT, nt = min(TT, t1 - ta);
    for (int i = tid; i < nt * dk; i += NT) {
      const int tt = i / dk, r = i - tt * dk;
      const float* row = qkv + (size_t)(ta + tt) * ld;
      delta_cp4(base + tt * DKP + r, row + k_off + kvh * dk + r);
      delta_cp4(base + TT * DKP + tt * DKP + r, row + q_off + kvh * dk + r);
    }
    for (int i = tid; i < nt * n_cols; i += NT) {
      const int tt = i / n_cols, cc = i - tt * n_cols;
      delta_cp4(base + 2 * TT * DKP + tt * DELTA_COLS + cc, qkv + (size_t)(ta + tt) * ld + v_off + h * dv + j0 + cc);
    }
    if (tid < nt) {
      delta_cp4(base + 2 * TT * DKP + TT * DELTA_COLS + tid, decay + (size_t)(ta + tid) * H + h);
      delta_cp4(base + 2 * TT * DKP + TT * DELTA_COLS + TT + tid, beta + (size_t)(ta + tid) * H + h);
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
    const float* ks = sm + buf * STAGE;
    const float* qs = ks + TT * DKP;
    const float* vs = qs + TT * DKP;
    const float* gs = vs + TT * DELTA_COLS;
    const float* bs = gs + TT;
    const int ta = t0 + tile * TT, nt = min(TT, t1 - ta);
    for (int tt = 0; tt < nt; tt++) {
      const float g = gs[tt], bt = bs[tt], v = vs[tt * DELTA_COLS + c];
      float kk[DKQ];
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int i = 0; i < DKQ; i += 2) {
        kk[i] = ks[tt * DKP + s + i * NS];
        kk[i + 1] = ks[tt * DKP + s + (i + 1) * NS];
        d0 = fmaf(S[i], kk[i], d0);
        d1 = fmaf(S[i + 1], kk[i + 1], d1);
      }
      float dot = d0 + d1;
#pragma unroll
      for (int o = 1; o < NS; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = bt * (v - g * dot);               // (g S)^T k = g (S^T k)
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int i = 0; i < DKQ; i += 2) {
        S[i] = fmaf(kk[i], u, g * S[i]);
        S[i + 1] = fmaf(kk[i + 1], u, g * S[i + 1]);
        o0 = fmaf(S[i], qs[tt * DKP + s + i * NS], o0);
        o1 = fmaf(S[i + 1], qs[tt * DKP + s + (i + 1) * NS], o1);
      }
      float out = o0 + o1;
#pragma unroll
      for (int o = 1; o < NS; o <<= 1) out += __shfl_xor_sync(0xffffffffu, out, o);
      if (s == 0 && col_ok) y[(size_t)(ta + tt) * ldy + h * dv + j] = out;
    }
    __syncthreads();                                    // the tile's buffer is free for the tile after the next
  }
  delta_cp_wait<0>();
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < DKQ; i++) {
      const int r = s + i * NS;
      if (r < dk) st[(size_t)r * dv] = S[i];
    }
  }
}

static int g_delta_split = 0;
// Fixes how many threads share a column of the state (4 or 8; 0: chosen from the key size); for tests and comparisons.
extern "C" void tlc_delta_rule_split(int threads) { g_delta_split = (threads == 4 || threads == 8) ? threads : 0; }

// qkv float [T, ld]: the normalised queries (G heads of dk) at q_off, keys at k_off, values (H heads of dv) at v_off;
// beta, decay float [T, H]; state float [n_slots, H, dk, dv], updated in place (a sequence at position 0 starts from
// zero whatever its slot holds); y float [T, ldy] receives o, head h at column h * dv.
extern "C" int tlc_delta_rule(const float* qkv, int ld, int q_off, int k_off, int v_off, const float* beta, const float* decay,
                              float* state, const int* cu_seqlens, const int* slots, const int* start_pos, int B, int H, int G,
                              int dk, int dv, float* y, int ldy, cudaStream_t stream) {
  if (B == 0) return 0;
  TLC_REQUIRE(H >= 1 && G >= 1 && H % G == 0 && H <= 65535 && B <= 65535, "delta_rule: %d heads over %d query/key heads, %d sequences", H, G, B);
  TLC_REQUIRE(dk >= 1 && dk <= 256 && dv >= 1, "delta_rule: keys of %d values exceed the kernel's limit of 256", dk);
  const dim3 grid((dv + DELTA_COLS - 1) / DELTA_COLS, H, B);
#define DELTA_LAUNCH(DKQ, NS, TT)                                                                                           \
  tlc_launch(delta_rule_kernel<DKQ, NS, TT>, grid, dim3(DELTA_COLS * NS), 0, stream, qkv, ld, q_off, k_off, v_off, beta, decay, state, \
             cu_seqlens, slots, start_pos, H, G, dk, dv, y, ldy)
  // threads a column: four, unless told otherwise.  Eight halve a token's chains of multiply-adds and give an SM's
  // schedulers a second warp, but measured no faster for prompts (2,048 tokens, 16 heads of 128 x 128: 829 against 837
  // us) and slower for single tokens (38 against 29 us at batch 64: one more round of shuffles)
  const int ns = g_delta_split ? g_delta_split : 4;
  if (dk <= 32) { if (ns == 4) DELTA_LAUNCH(8, 4, 16); else DELTA_LAUNCH(4, 8, 16); }
  else if (dk <= 64) { if (ns == 4) DELTA_LAUNCH(16, 4, 16); else DELTA_LAUNCH(8, 8, 16); }
  else if (dk <= 128) { if (ns == 4) DELTA_LAUNCH(32, 4, 16); else DELTA_LAUNCH(16, 8, 16); }
  else DELTA_LAUNCH(32, 8, 8);
#undef DELTA_LAUNCH
  TLC_CHECK_LAUNCH("delta_rule");
  return 0;
}
