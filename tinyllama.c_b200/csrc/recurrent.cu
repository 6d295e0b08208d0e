// minGRU: a recurrence whose update gate and candidate depend on the token's input alone, never on the previous state.
//
// Per channel, with the projections zr, ur, gr of the token (biases already added):
//   z = sigmoid(zr);  cand = ur + 1/2 where ur >= 0, sigmoid(ur) where ur < 0;  S <- (1 - z) S + z cand;
//   y = S * silu(gr).
// S starts at zero, is 32-bit and lives in the sequence's slot of `state` [n_slots, W] between steps.  Everything here
// is 32-bit; only y takes the activation type (a bfloat16 run takes the quick exponential and reciprocal).  The recurrence is linear in S (S <- a S + b with a = 1 - z, b = z cand),
// so a long prompt is cut into chunks that run side by side: every chunk first reduces to its (product of a, end value
// from zero), a walk over a sequence's chunks turns those into the state each chunk starts from, and the chunks then
// run again from there and write their outputs.
#include "common.cuh"

// QUICK (bfloat16 runs): exponential and reciprocal by the special-function unit, a few units in the last place of 32 bits;
// 32-bit runs divide in full precision.
template <bool QUICK> __device__ __forceinline__ float sigmoid_of(float x) {
  return QUICK ? __fdividef(1.0f, 1.0f + __expf(-x)) : 1.0f / (1.0f + expf(-x));
}

struct GruStep { float a, b; };
template <bool QUICK> __device__ __forceinline__ GruStep gru_step(float zr, float ur) {
  const float z = sigmoid_of<QUICK>(zr);
  const float cand = ur >= 0.f ? ur + 0.5f : sigmoid_of<QUICK>(ur);
  GruStep s;
  s.a = 1.0f - z;
  s.b = z * cand;
  return s;
}

// One thread per (sequence, channel) walks the sequence's rows of this step.
template <typename TO, bool QUICK>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(const float* __restrict__ proj, int ld, int z_off, int u_off, int g_off, int W, float* state,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ slots, const int* __restrict__ start_pos,
                   TO* __restrict__ out, int out_ld) {
  tlc_pdl(proj, state, out);
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= W) return;
  float* st = state + (size_t)slots[b] * W + c;
  float S = start_pos[b] == 0 ? 0.f : *st;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  for (int t = t0; t < t1; t++) {
    const float* pr = proj + (size_t)t * ld;
    const GruStep s = gru_step<QUICK>(pr[z_off + c], pr[u_off + c]);
    S = fmaf(s.a, S, s.b);
    out[(size_t)t * out_ld + c] = from_f32<TO>(S * silu_of<QUICK>(pr[g_off + c]));
  }
  *st = S;
}

// Chunked form, pass 1: chunk j reduces to pa[j, c] = product of a and pb[j, c] = its end value from zero.
template <bool QUICK>
__global__ void __launch_bounds__(128)
mingru_chunk_reduce_kernel(const float* __restrict__ proj, int ld, int z_off, int u_off, int W,
                           const int* __restrict__ seg_start, float* __restrict__ pa, float* __restrict__ pb) {
  tlc_pdl(proj, pa, pb);
  const int j = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int t0 = seg_start[j], t1 = seg_start[j + 1];
  float A = 1.0f, S = 0.f;
  for (int t = t0; t < t1; t++) {
    const float* pr = proj + (size_t)t * ld;
    const GruStep s = gru_step<QUICK>(pr[z_off + c], pr[u_off + c]);
    S = fmaf(s.a, S, s.b);
    A *= s.a;
  }
  pa[(size_t)j * W + c] = A;
  pb[(size_t)j * W + c] = S;
}

// Pass 2: a thread per (sequence, channel) walks the sequence's chunks; pb[j] becomes the state chunk j starts from,
// and the slot receives the state after the last chunk.
__global__ void __launch_bounds__(128)
mingru_chunk_carry_kernel(const float* __restrict__ pa, float* __restrict__ pb, int W, float* state,
                          const int* __restrict__ seq_seg_start, const int* __restrict__ slots,
                          const int* __restrict__ start_pos) {
  tlc_pdl(pa, pb, state);
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= W) return;
  float* st = state + (size_t)slots[b] * W + c;
  float S = start_pos[b] == 0 ? 0.f : *st;
  for (int j = seq_seg_start[b]; j < seq_seg_start[b + 1]; j++) {
    const float A = pa[(size_t)j * W + c], E = pb[(size_t)j * W + c];
    pb[(size_t)j * W + c] = S;
    S = fmaf(A, S, E);
  }
  *st = S;
}

// Pass 3: every chunk again, from its true start state, with outputs.
template <typename TO, bool QUICK>
__global__ void __launch_bounds__(128)
mingru_chunk_apply_kernel(const float* __restrict__ proj, int ld, int z_off, int u_off, int g_off, int W,
                          const int* __restrict__ seg_start, const float* __restrict__ s_in, TO* __restrict__ out, int out_ld) {
  tlc_pdl(proj, s_in, out);
  const int j = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int t0 = seg_start[j], t1 = seg_start[j + 1];
  float S = s_in[(size_t)j * W + c];
  for (int t = t0; t < t1; t++) {
    const float* pr = proj + (size_t)t * ld;
    const GruStep s = gru_step<QUICK>(pr[z_off + c], pr[u_off + c]);
    S = fmaf(s.a, S, s.b);
    out[(size_t)t * out_ld + c] = from_f32<TO>(S * silu_of<QUICK>(pr[g_off + c]));
  }
}

extern "C" int tlc_mingru_scan(const float* proj, int ld, int z_off, int u_off, int g_off, int W, float* state,
                               const int* cu_seqlens, const int* slots, const int* start_pos, int B, void* out, int out_dtype,
                               int out_ld, const int* seg_start, const int* seq_seg_start, int n_seg, float* scratch,
                               cudaStream_t stream) {
  if (B == 0 || W == 0) return 0;
  const unsigned cy = (unsigned)((W + 127) / 128);
  if (seg_start == nullptr || n_seg <= 0) {
    if (out_dtype == TLC_BF16)
      tlc_launch(mingru_scan_kernel<__nv_bfloat16, true>, dim3(B, cy), dim3(128), 0, stream, proj, ld, z_off, u_off, g_off, W, state,
                 cu_seqlens, slots, start_pos, (__nv_bfloat16*)out, out_ld);
    else
      tlc_launch(mingru_scan_kernel<float, false>, dim3(B, cy), dim3(128), 0, stream, proj, ld, z_off, u_off, g_off, W, state,
                 cu_seqlens, slots, start_pos, (float*)out, out_ld);
    TLC_CHECK_LAUNCH("mingru_scan");
    return 0;
  }
  TLC_REQUIRE(scratch != nullptr && seq_seg_start != nullptr, "mingru_scan: the chunked form needs its tables and 2 * n_seg * W floats");
  float* pa = scratch;
  float* pb = scratch + (size_t)n_seg * W;
  if (out_dtype == TLC_BF16)
    tlc_launch(mingru_chunk_reduce_kernel<true>, dim3(n_seg, cy), dim3(128), 0, stream, proj, ld, z_off, u_off, W, seg_start, pa, pb);
  else
    tlc_launch(mingru_chunk_reduce_kernel<false>, dim3(n_seg, cy), dim3(128), 0, stream, proj, ld, z_off, u_off, W, seg_start, pa, pb);
  TLC_CHECK_LAUNCH("mingru_chunk_reduce");
  tlc_launch(mingru_chunk_carry_kernel, dim3(B, cy), dim3(128), 0, stream, (const float*)pa, pb, W, state, seq_seg_start, slots,
             start_pos);
  TLC_CHECK_LAUNCH("mingru_chunk_carry");
  if (out_dtype == TLC_BF16)
    tlc_launch(mingru_chunk_apply_kernel<__nv_bfloat16, true>, dim3(n_seg, cy), dim3(128), 0, stream, proj, ld, z_off, u_off, g_off, W,
               seg_start, (const float*)pb, (__nv_bfloat16*)out, out_ld);
  else
    tlc_launch(mingru_chunk_apply_kernel<float, false>, dim3(n_seg, cy), dim3(128), 0, stream, proj, ld, z_off, u_off, g_off, W,
               seg_start, (const float*)pb, (float*)out, out_ld);
  TLC_CHECK_LAUNCH("mingru_chunk_apply");
  return 0;
}
