// delta.cu — the gated delta rule mixer of a model given as a list of layers
// (nvllm_mixer_kind NVLLM_MIXER_DELTA), for a ragged batch of sequences, between its two
// projections (ordinary GEMMs, forward_layered.cu).
//
// Per head, with a dim x vdim state S kept in fp32 per state slot, for every token in order:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// q, k (kv_heads x dim, shared by heads / kv_heads heads each) and v (heads x vdim) come from
// the fused input projection through a causal convolution over time per channel (taps from the
// layer, zeros before the sequence start, the last column is the current token's), SiLU, and for
// q / k a division by the head's Euclidean length (eps 1e-6 under the root; q also by sqrt(dim)).
// beta = sigmoid(W_b x), g = exp(-exp(A_log) softplus(W_a x + dt_bias)) per head.  The read-out
// of a head is divided by its root mean square over vdim, multiplied by a weight shared by the
// heads and by silu(W_g x), and goes to the output projection.
//
//   delta_prep_kernel  per token: split-K sum of the projection, convolution (the taps - 1
//                      inputs before the step's first token come from the slot's tail), SiLU,
//                      unit lengths; beta and g.  All fp32.
//   delta_scan_kernel  one CTA per (sequence, head, block of value columns).  A value column of
//                      the state is independent of the others: it lives in the registers of LPC
//                      lanes (dim / LPC entries each), the two inner products of a token are
//                      reduced with shuffles inside that lane group.  Token inputs arrive in
//                      double-buffered shared-memory tiles of 16 tokens (cp.async), so the loop
//                      over tokens never waits for memory.  The state is read from the slot when
//                      the sequence has earlier tokens (zero otherwise) and written back at the
//                      end; the sequence's CTAs also roll the convolution tail forward.
//   delta_out_kernel   one CTA per token, a warp per head: RMS over vdim, weight, gate -> act dtype.
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "mma.cuh"

namespace nvllm {

namespace {
__device__ __forceinline__ int seq_of_row(const int* __restrict__ cu_q, int n_seqs, int row) {
  int lo = 0, hi = n_seqs - 1;  // last s with cu_q[s] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= row) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}
__device__ __forceinline__ float sum_slices(const float* __restrict__ p, int S, size_t stride) {
  float acc = 0.f;
  for (int s = 0; s < S; s++) acc += p[(size_t)s * stride];
  return acc;
}
__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
// SiLU of the convolution outputs and of the output gate: exact in the fp32 mode, fast
// intrinsics (relative error about 1e-6, far below the bf16 rounding that follows) otherwise
template <bool FAST>
__device__ __forceinline__ float silu_t(float x) {
  return FAST ? __fdividef(x, 1.0f + __expf(-x)) : silu(x);
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
}  // namespace

constexpr int DELTA_MAX_TAPS = 8;

// grid (T, Y), 256 threads.  The channels of a row are cut into units that a WARP finishes on
// its own: the G query heads, the G key heads (a unit = one head, whose length the warp needs)
// and the value channels in pieces of 32 * MAXV; the warps of the row's CTAs take the units in
// turn.  A lane holds up to MAXV channels of its unit; all their taps' loads are in flight at once.
template <int MAXV, bool FAST>
__global__ void __launch_bounds__(256) delta_prep_kernel(DeltaArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  // one row per sequence (a decode step): row t is sequence t, no search through the offsets
  const int s = a.T == a.n_seqs ? t : seq_of_row(a.cu_q, a.n_seqs, t);
  const int r0 = a.cu_q[s];
  const int li = t - r0;                 // index among the step's rows of the sequence
  const int pos = a.positions[r0] + li;  // position in the sequence
  const float* tail = a.state_pool + (size_t)a.state_slots[s] * a.slot_floats + a.tail_off;  // [taps - 1][conv_ch]
  constexpr int PIECE = 32 * MAXV;
  const int v_units = ceil_div(a.n_v, PIECE);
  const int n_units = 2 * a.G + v_units;
  const float qmul = 1.0f / sqrtf((float)a.dim);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int u = blockIdx.y * nw + warp; u < n_units; u += gridDim.y * nw) {
    const bool head = u < 2 * a.G;
    const int c0 = head ? u * a.dim : a.n_q + a.n_k + (u - 2 * a.G) * PIECE;
    const int cn = head ? a.dim : min(PIECE, a.conv_ch - c0);
    float val[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; i++) val[i] = 0.f;
    for (int k = 0; k < a.taps; k++) {  // tap k reads the token taps - 1 - k positions earlier
      const int back = a.taps - 1 - k;
      const float* src = nullptr;
      int S = 1;
      size_t stride = 0;
      if (li - back >= 0) { src = a.in_p + (size_t)(t - back) * a.in_ld; S = a.in_S; stride = a.in_stride; }
      else if (pos - back >= 0) src = tail + (size_t)(a.taps - 1 + li - back) * a.conv_ch;
      if (!src) continue;  // before the start of the sequence: zeros
#pragma unroll
      for (int i = 0; i < MAXV; i++) {
        const int c = c0 + lane + 32 * i;
        if (lane + 32 * i < cn) val[i] = fmaf(sum_slices(src + c, S, stride), a.conv_w[c * a.taps + k], val[i]);
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
      val[i] = (lane + 32 * i < cn) ? silu_t<FAST>(val[i]) : 0.f;
      ss += val[i] * val[i];
    }
    float mul = 1.f;
    if (head) {  // unit length; the queries also carry 1 / sqrt(dim)
      mul = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
      if (u < a.G) mul *= qmul;
    }
#pragma unroll
    for (int i = 0; i < MAXV; i++)
      if (lane + 32 * i < cn) a.qkv[(size_t)t * a.conv_ch + c0 + lane + 32 * i] = val[i] * mul;
  }
  if (blockIdx.y == 0 && threadIdx.x < a.H) {
    const int h = threadIdx.x;
    const float* p = a.in_p + (size_t)t * a.in_ld + a.conv_ch;
    const float b = sum_slices(p + h, a.in_S, a.in_stride);
    const float d = sum_slices(p + a.H + h, a.in_S, a.in_stride);
    a.bg[(size_t)t * 2 * a.H + h] = 1.0f / (1.0f + expf(-b));
    a.bg[(size_t)t * 2 * a.H + a.H + h] = expf(-expf(a.a_log[h]) * softplus(d + a.dt_bias[h]));
  }
  TRACE_EXIT(tr);
}

cudaError_t launch_delta_prep(cudaStream_t st, const DeltaArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (a.taps < 1 || a.taps > DELTA_MAX_TAPS || a.H > 256 || a.dim > 1024) return cudaErrorInvalidValue;
  const int maxv = a.dim <= 128 ? 4 : a.dim <= 256 ? 8 : 32;
  const int n_units = 2 * a.G + ceil_div(a.n_v, 32 * maxv);
  // few rows (decode): a row's units spread over several CTAs
  const int ny = a.T >= 2048 ? 1 : std::min(ceil_div(n_units, 8), std::max(1, 2048 / a.T));
  const dim3 grid(a.T, ny);
  if (a.fast_act) {
    if (maxv == 4) (void)launch_k(delta_prep_kernel<4, true>, grid, dim3(256), 0, st, a, next_trace(34));
    else if (maxv == 8) (void)launch_k(delta_prep_kernel<8, true>, grid, dim3(256), 0, st, a, next_trace(34));
    else (void)launch_k(delta_prep_kernel<32, true>, grid, dim3(256), 0, st, a, next_trace(34));
  } else {
    if (maxv == 4) (void)launch_k(delta_prep_kernel<4, false>, grid, dim3(256), 0, st, a, next_trace(34));
    else if (maxv == 8) (void)launch_k(delta_prep_kernel<8, false>, grid, dim3(256), 0, st, a, next_trace(34));
    else (void)launch_k(delta_prep_kernel<32, false>, grid, dim3(256), 0, st, a, next_trace(34));
  }
  return cudaGetLastError();
}

// ------------------------------------------------------------------ scan
constexpr int DELTA_TT = 16;  // tokens per shared-memory tile

// block = VC * LPC threads: thread (jl = tid / LPC, p = tid % LPC) holds rows d = r * LPC + p,
// r < R, of value column vbase + jl
template <int R>
__global__ void __launch_bounds__(256) delta_scan_kernel(DeltaArgs a, int LPC, int VC, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int dim = a.dim, vdim = a.vdim;
  const int s = blockIdx.x, h = blockIdx.y, vbase = blockIdx.z * VC;
  const int r0 = a.cu_q[s], r1 = a.cu_q[s + 1];
  const int n_new = r1 - r0;
  const int start = a.positions[r0];
  float* slot = a.state_pool + (size_t)a.state_slots[s] * a.slot_floats;
  const int tid = threadIdx.x;
  const int p = tid % LPC, jl = tid / LPC;
  const int col = vbase + jl;
  const bool col_ok = jl < VC && col < vdim;
  const int kvh = h / (a.H / a.G);

  // convolution tail of the slot: after this step it holds the inputs of the last taps - 1
  // positions.  The sequence's CTAs share the channels, a thread per channel, old values read
  // before any write (the prep kernel, which also reads the tail, finished before this kernel's wait).
  if (a.taps > 1) {
    float* tail = slot + a.tail_off;
    const int part = h * gridDim.z + blockIdx.z, parts = a.H * gridDim.z;  // the sequence's CTAs share the channels
    for (int c = part * blockDim.x + tid; c < a.conv_ch; c += parts * blockDim.x) {
      float nv[DELTA_MAX_TAPS];
#pragma unroll
      for (int j = 0; j < DELTA_MAX_TAPS - 1; j++) {
        if (j >= a.taps - 1) break;
        const int q = n_new - (a.taps - 1) + j;  // row of the step that lands in tail[j]; < 0: an older input
        if (q >= 0) nv[j] = sum_slices(a.in_p + (size_t)(r0 + q) * a.in_ld + c, a.in_S, a.in_stride);
        else nv[j] = (start + q >= 0) ? tail[(size_t)(j + n_new) * a.conv_ch + c] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < DELTA_MAX_TAPS - 1; j++) {
        if (j >= a.taps - 1) break;
        tail[(size_t)j * a.conv_ch + c] = nv[j];
      }
    }
  }

  float* S_g = slot + a.state_off + (size_t)h * dim * vdim;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; r++) {
    const int d = r * LPC + p;
    S[r] = (start > 0 && col_ok && d < dim) ? S_g[(size_t)d * vdim + col] : 0.f;
  }
  // tile of DELTA_TT tokens: q [TT][dim], k [TT][dim], v [TT][VC], beta [TT], g [TT]
  const int tile_floats = DELTA_TT * (2 * dim + VC + 2);
  const float* qg = a.qkv + (size_t)kvh * dim;
  const float* kg = a.qkv + a.n_q + (size_t)kvh * dim;
  const float* vg = a.qkv + a.n_q + a.n_k + (size_t)h * vdim + vbase;
  const int vcn = min(VC, vdim - vbase);
  auto issue = [&](int t0, int buf) {
    float* b = sm + buf * tile_floats;
    const int nt = min(DELTA_TT, n_new - t0);
    const uint32_t qb = smem_addr(b), kb = smem_addr(b + DELTA_TT * dim), vb = smem_addr(b + 2 * DELTA_TT * dim),
                   bb = smem_addr(b + DELTA_TT * (2 * dim + VC));
    for (int i = tid; i < nt * dim; i += blockDim.x) {
      const int tt = i / dim, d = i % dim;
      const size_t rowo = (size_t)(r0 + t0 + tt) * a.conv_ch;
      cp_async4(qb + 4 * i, qg + rowo + d);
      cp_async4(kb + 4 * i, kg + rowo + d);
    }
    for (int i = tid; i < nt * vcn; i += blockDim.x) {
      const int tt = i / vcn, j = i % vcn;
      cp_async4(vb + 4 * (tt * VC + j), vg + (size_t)(r0 + t0 + tt) * a.conv_ch + j);
    }
    for (int i = tid; i < nt * 2; i += blockDim.x) {
      const int tt = i >> 1, w = i & 1;
      cp_async4(bb + 4 * (w * DELTA_TT + tt), a.bg + (size_t)(r0 + t0 + tt) * 2 * a.H + w * a.H + h);
    }
  };
  issue(0, 0);
  cp_async_commit();
  float* og = a.o + (size_t)h * vdim + col;
  const int HV = a.H * vdim;
  for (int t0 = 0, it = 0; t0 < n_new; t0 += DELTA_TT, it++) {
    const int buf = it & 1;
    if (t0 + DELTA_TT < n_new) issue(t0 + DELTA_TT, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* b = sm + buf * tile_floats;
    const float* qs = b;
    const float* ks = b + DELTA_TT * dim;
    const float* vs = b + 2 * DELTA_TT * dim;
    const float* bs = b + DELTA_TT * (2 * dim + VC);
    const int nt = min(DELTA_TT, n_new - t0);
    for (int tt = 0; tt < nt; tt++) {
      const float beta = bs[tt], g = bs[DELTA_TT + tt];
      const float v = col_ok ? vs[tt * VC + jl] : 0.f;
      float kr[R];
      float dot = 0.f;
#pragma unroll
      for (int r = 0; r < R; r++) {
        const int d = r * LPC + p;
        kr[r] = d < dim ? ks[tt * dim + d] : 0.f;
        S[r] *= g;
        dot = fmaf(S[r], kr[r], dot);
      }
      for (int o = 1; o < LPC; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = beta * (v - dot);
      float out = 0.f;
#pragma unroll
      for (int r = 0; r < R; r++) {
        const int d = r * LPC + p;
        S[r] = fmaf(kr[r], u, S[r]);
        const float qv = d < dim ? qs[tt * dim + d] : 0.f;
        out = fmaf(S[r], qv, out);
      }
      for (int o = 1; o < LPC; o <<= 1) out += __shfl_xor_sync(0xffffffffu, out, o);
      if (p == 0 && col_ok) og[(size_t)(r0 + t0 + tt) * HV] = out;
    }
    __syncthreads();  // the buffer may be refilled
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < R; r++) {
    const int d = r * LPC + p;
    if (col_ok && d < dim) S_g[(size_t)d * vdim + col] = S[r];
  }
  TRACE_EXIT(tr);
}


// The same scan with compile-time sizes, dim = R * LPC: lane p of a column holds the R
// neighbouring rows p R .. p R + R - 1, the keys and queries of a token sit in shared memory as
// LPC segments of R + 4 floats (the padding puts the lanes' 16-byte reads in different banks),
// no bounds checks in the token loop, four partial sums per inner product; one column per
// thread and two CTAs per SM, or two columns per thread (CC = 2) and one.
template <int R, int LPC, int CC>
__global__ void __launch_bounds__(256, CC == 1 ? 2 : 1) delta_scan_fixed_kernel(DeltaArgs a, int VC, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  constexpr int DIM = R * LPC, RP = R + 4, KL = LPC * RP;
  const int vdim = a.vdim;
  const int s = blockIdx.x, h = blockIdx.y, vbase = blockIdx.z * VC;
  const int r0 = a.cu_q[s], r1 = a.cu_q[s + 1];
  const int n_new = r1 - r0;
  const int start = a.positions[r0];
  float* slot = a.state_pool + (size_t)a.state_slots[s] * a.slot_floats;
  const int tid = threadIdx.x;
  const int p = tid % LPC, jl = tid / LPC;  // the thread's CC columns: vbase + jl + cc * (VC / CC)
  const int VH = VC / CC;
  bool col_ok[CC];
  int col[CC];
#pragma unroll
  for (int cc = 0; cc < CC; cc++) {
    col[cc] = vbase + jl + cc * VH;
    col_ok[cc] = jl < VH && col[cc] < vdim;
  }
  const int kvh = h / (a.H / a.G);

  if (a.taps > 1) {  // roll the convolution tail forward (see the generic kernel)
    float* tail = slot + a.tail_off;
    const int part = h * gridDim.z + blockIdx.z, parts = a.H * gridDim.z;
    for (int c = part * blockDim.x + tid; c < a.conv_ch; c += parts * blockDim.x) {
      float nv[DELTA_MAX_TAPS];
#pragma unroll
      for (int j = 0; j < DELTA_MAX_TAPS - 1; j++) {
        if (j >= a.taps - 1) break;
        const int q = n_new - (a.taps - 1) + j;
        if (q >= 0) nv[j] = sum_slices(a.in_p + (size_t)(r0 + q) * a.in_ld + c, a.in_S, a.in_stride);
        else nv[j] = (start + q >= 0) ? tail[(size_t)(j + n_new) * a.conv_ch + c] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < DELTA_MAX_TAPS - 1; j++) {
        if (j >= a.taps - 1) break;
        tail[(size_t)j * a.conv_ch + c] = nv[j];
      }
    }
  }

  float* S_g = slot + a.state_off + (size_t)h * DIM * vdim;
  float S[CC][R];
#pragma unroll
  for (int cc = 0; cc < CC; cc++)
#pragma unroll
    for (int r = 0; r < R; r++) S[cc][r] = (start > 0 && col_ok[cc]) ? S_g[(size_t)(p * R + r) * vdim + col[cc]] : 0.f;
  // tile of DELTA_TT tokens: q [TT][KL], k [TT][KL], v [TT][VC], beta [TT], g [TT]
  const int tile_floats = DELTA_TT * (2 * KL + VC + 2);
  const float* qg = a.qkv + (size_t)kvh * DIM;
  const float* kg = a.qkv + a.n_q + (size_t)kvh * DIM;
  const float* vg = a.qkv + a.n_q + a.n_k + (size_t)h * vdim + vbase;
  const int vcn = min(VC, vdim - vbase);
  auto issue = [&](int t0, int buf) {
    float* b = sm + buf * tile_floats;
    const int nt = min(DELTA_TT, n_new - t0);
    const uint32_t qb = smem_addr(b), kb = smem_addr(b + DELTA_TT * KL), vb = smem_addr(b + 2 * DELTA_TT * KL),
                   bb = smem_addr(b + DELTA_TT * (2 * KL + VC));
    for (int i = tid; i < nt * (DIM / 4); i += blockDim.x) {  // 16 bytes at a time: rows and segments are 16-byte aligned
      const int tt = i / (DIM / 4), d = (i % (DIM / 4)) * 4;
      const size_t rowo = (size_t)(r0 + t0 + tt) * a.conv_ch;
      const int so = tt * KL + (d / R) * RP + d % R;
      cp_async16(qb + 4 * so, qg + rowo + d, true);
      cp_async16(kb + 4 * so, kg + rowo + d, true);
    }
    for (int i = tid; i < nt * vcn; i += blockDim.x) {
      const int tt = i / vcn, j = i % vcn;
      cp_async4(vb + 4 * (tt * VC + j), vg + (size_t)(r0 + t0 + tt) * a.conv_ch + j);
    }
    for (int i = tid; i < nt * 2; i += blockDim.x) {
      const int tt = i >> 1, w = i & 1;
      cp_async4(bb + 4 * (w * DELTA_TT + tt), a.bg + (size_t)(r0 + t0 + tt) * 2 * a.H + w * a.H + h);
    }
  };
  issue(0, 0);
  cp_async_commit();
  const int HV = a.H * vdim;
  float* og = a.o + (size_t)h * vdim;
  for (int t0 = 0, it = 0; t0 < n_new; t0 += DELTA_TT, it++) {
    const int buf = it & 1;
    if (t0 + DELTA_TT < n_new) issue(t0 + DELTA_TT, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* b = sm + buf * tile_floats;
    const float* qs = b + p * RP;
    const float* ks = b + DELTA_TT * KL + p * RP;
    const float* vs = b + 2 * DELTA_TT * KL;
    const float* bs = b + DELTA_TT * (2 * KL + VC);
    const int nt = min(DELTA_TT, n_new - t0);
    for (int tt = 0; tt < nt; tt++) {
      const float beta = bs[tt], g = bs[DELTA_TT + tt];
      float v[CC], dot[CC], out[CC];
#pragma unroll
      for (int cc = 0; cc < CC; cc++) v[cc] = col_ok[cc] ? vs[tt * VC + jl + cc * VH] : 0.f;
      float kr[R];
      float d4[CC][4];
#pragma unroll
      for (int cc = 0; cc < CC; cc++) d4[cc][0] = d4[cc][1] = d4[cc][2] = d4[cc][3] = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + tt * KL + r);
        kr[r] = k4.x; kr[r + 1] = k4.y; kr[r + 2] = k4.z; kr[r + 3] = k4.w;
#pragma unroll
        for (int cc = 0; cc < CC; cc++)
#pragma unroll
          for (int e = 0; e < 4; e++) {
            S[cc][r + e] *= g;
            d4[cc][e] = fmaf(S[cc][r + e], kr[r + e], d4[cc][e]);
          }
      }
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        dot[cc] = (d4[cc][0] + d4[cc][1]) + (d4[cc][2] + d4[cc][3]);
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1) dot[cc] += __shfl_xor_sync(0xffffffffu, dot[cc], o);
        dot[cc] = beta * (v[cc] - dot[cc]);  // u: what the token writes into the column
        d4[cc][0] = d4[cc][1] = d4[cc][2] = d4[cc][3] = 0.f;
      }
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qs + tt * KL + r);
        const float qv[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int cc = 0; cc < CC; cc++)
#pragma unroll
          for (int e = 0; e < 4; e++) {
            S[cc][r + e] = fmaf(kr[r + e], dot[cc], S[cc][r + e]);
            d4[cc][e] = fmaf(S[cc][r + e], qv[e], d4[cc][e]);
          }
      }
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        out[cc] = (d4[cc][0] + d4[cc][1]) + (d4[cc][2] + d4[cc][3]);
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1) out[cc] += __shfl_xor_sync(0xffffffffu, out[cc], o);
        if (p == 0 && col_ok[cc]) og[(size_t)(r0 + t0 + tt) * HV + col[cc]] = out[cc];
      }
    }
    __syncthreads();  // the buffer may be refilled
  }
  cp_async_wait<0>();
#pragma unroll
  for (int cc = 0; cc < CC; cc++)
    if (col_ok[cc]) {
#pragma unroll
      for (int r = 0; r < R; r++) S_g[(size_t)(p * R + r) * vdim + col[cc]] = S[cc][r];
    }
  TRACE_EXIT(tr);
}

template <int R, int LPC>
static cudaError_t delta_scan_fixed_launch(cudaStream_t st, const DeltaArgs& a) {
  // two columns per thread (the key / query reads from shared memory, which bound the one-column
  // form, serve both) when the head has the columns for it
  static const bool cc2_on = !(getenv("NVLLM_DELTA_CC2") && atoi(getenv("NVLLM_DELTA_CC2")) == 0);
  const bool cc2 = cc2_on && a.vdim >= 2 * (256 / LPC);
  int VC = (cc2 ? 2 : 1) * (256 / LPC);
  if (VC > a.vdim) VC = a.vdim;
  const int threads = cc2 ? 256 : (VC * LPC + 31) / 32 * 32;
  const dim3 grid(a.n_seqs, a.H, ceil_div(a.vdim, VC));
  const size_t smem = (size_t)2 * DELTA_TT * (2 * LPC * (R + 4) + VC + 2) * sizeof(float);
  if (cc2) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(delta_scan_fixed_kernel<R, LPC, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(delta_scan_fixed_kernel<R, LPC, 2>, grid, dim3(threads), smem, st, a, VC, next_trace(35));
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(delta_scan_fixed_kernel<R, LPC, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(delta_scan_fixed_kernel<R, LPC, 1>, grid, dim3(threads), smem, st, a, VC, next_trace(35));
  }
  return cudaGetLastError();
}

cudaError_t launch_delta_scan(cudaStream_t st, const DeltaArgs& a) {
  if (a.n_seqs <= 0) return cudaSuccess;
  if (a.dim > 1024 || a.H % a.G) return cudaErrorInvalidValue;
  // compile-time sizes for the usual head widths (rows of the step's inputs must be 16-byte aligned)
  static const bool fixed_on = !(getenv("NVLLM_DELTA_FIXED") && atoi(getenv("NVLLM_DELTA_FIXED")) == 0);
  if (fixed_on && a.conv_ch % 4 == 0 && a.n_q % 4 == 0 && a.n_k % 4 == 0) {
    switch (a.dim) {
      case 16: return delta_scan_fixed_launch<4, 4>(st, a);
      case 32: return delta_scan_fixed_launch<8, 4>(st, a);
      case 48: return delta_scan_fixed_launch<12, 4>(st, a);
      case 64: return delta_scan_fixed_launch<16, 4>(st, a);
      case 96: return delta_scan_fixed_launch<24, 4>(st, a);
      case 128: return delta_scan_fixed_launch<32, 4>(st, a);
      case 256: return delta_scan_fixed_launch<32, 8>(st, a);
    }
  }
  // registers per thread R and lanes per column LPC (a power of two): R * LPC >= dim
  int R = 4;
  while (R < 32 && R * 4 < a.dim) R *= 2;
  int LPC = 1;
  while (R * LPC < a.dim) LPC *= 2;
  int VC = 256 / LPC;
  if (VC > a.vdim) VC = a.vdim;
  int threads = VC * LPC;
  threads = (threads + 31) / 32 * 32;  // whole warps: every lane takes part in the shuffles
  const dim3 grid(a.n_seqs, a.H, ceil_div(a.vdim, VC));
  const size_t smem = (size_t)2 * DELTA_TT * (2 * a.dim + VC + 2) * sizeof(float);
#define DS(RR)                                                                                        \
  {                                                                                                   \
    if (smem > 48 * 1024)                                                                             \
      cudaFuncSetAttribute(delta_scan_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    (void)launch_k(delta_scan_kernel<RR>, grid, dim3(threads), smem, st, a, LPC, VC, next_trace(35));   \
  }
  if (R == 4) DS(4)
  else if (R == 8) DS(8)
  else if (R == 16) DS(16)
  else DS(32)
#undef DS
  return cudaGetLastError();
}

// ------------------------------------------------------------------ gated norm of the read-out
template <typename OT, int MV>
__global__ void __launch_bounds__(256) delta_out_kernel(DeltaArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int vdim = a.vdim;
  OT* out = (OT*)a.out + (size_t)t * a.o_ld;
  const float* gate = a.in_p + (size_t)t * a.in_ld + a.conv_ch + 2 * a.H;
  // heads of up to 32 * MV columns stay in registers: read-outs and gates are loaded together
  constexpr bool FAST = sizeof(OT) == 2;
  for (int h = blockIdx.y * nw + warp; h < a.H; h += gridDim.y * nw) {
    const float* o = a.o + (size_t)t * a.H * vdim + (size_t)h * vdim;
    if (vdim <= 32 * MV) {
      float ov[MV], gv[MV];
#pragma unroll
      for (int c = 0; c < MV; c++) {
        const int i = lane + 32 * c;
        ov[c] = i < vdim ? o[i] : 0.f;
        gv[c] = i < vdim ? sum_slices(gate + h * vdim + i, a.in_S, a.in_stride) : 0.f;
      }
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < MV; c++) ss += ov[c] * ov[c];
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + a.eps);
#pragma unroll
      for (int c = 0; c < MV; c++) {
        const int i = lane + 32 * c;
        if (i < vdim) out[h * vdim + i] = from_f32<OT>(ov[c] * inv * a.onorm_w[i] * silu_t<FAST>(gv[c]));
      }
      continue;
    }
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss += o[i] * o[i];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + a.eps);
    for (int i = lane; i < vdim; i += 32) {
      const float gt = sum_slices(gate + h * vdim + i, a.in_S, a.in_stride);
      out[h * vdim + i] = from_f32<OT>(o[i] * inv * a.onorm_w[i] * silu(gt));
    }
  }
  if (blockIdx.y == 0)
    for (int c = a.H * vdim + threadIdx.x; c < a.o_ld; c += blockDim.x) out[c] = from_f32<OT>(0.f);
  TRACE_EXIT(tr);
}

cudaError_t launch_delta_out(cudaStream_t st, int odt, const DeltaArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  const dim3 grid(a.T, a.T >= 1024 ? 1 : ceil_div(a.H, 8));  // few rows (decode): a row's heads spread over several CTAs
  if (odt == DT_F32) (void)launch_k(delta_out_kernel<float, 8>, grid, dim3(256), 0, st, a, next_trace(36));
  else if (a.vdim <= 128) (void)launch_k(delta_out_kernel<bf16, 4>, grid, dim3(256), 0, st, a, next_trace(36));
  else (void)launch_k(delta_out_kernel<bf16, 8>, grid, dim3(256), 0, st, a, next_trace(36));
  return cudaGetLastError();
}

}  // namespace nvllm
