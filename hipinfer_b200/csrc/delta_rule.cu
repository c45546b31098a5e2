// The generalized delta rule: a linear recurrence with a state matrix per head, carried from token to token.
//
// Per head, with state S [D key channels][D value channels] (32-bit, in a state slot of the request):
//     u  = k / sqrt(sum(k^2) + unit_eps)
//     S' = diag(w) S - (a * u) (u^T S) + k v^T          (both terms read the old state)
//     o  = S'^T r
//     w  = exp(-decay_scale * sigmoid(w_raw + w_bias)),   a = sigmoid(a_raw + a_bias)
// and then the head's output: o / sqrt(mean(o^2) + eps) * norm_weight * sigmoid(gate_raw).
// r, k, v, a_raw, gate_raw are columns of the 32-bit result of one projection, w_raw of another; everything here
// is 32-bit (expf, the sums, the state); the output is rounded once.
//
// Value channel j of the state, S[:, j], never meets another channel: u^T S and S^T r are sums over key channels.
// So a block owns (request, head) and its threads own value channels; the tokens of the request's portion run in
// order, the state stays on chip from the first to the last of them, and is written back once. Which requests
// and how many tokens comes from device arrays (first row, row count and state slot of each request), so the
// launch is the same for every batch of as many requests and replays from a CUDA graph.
//
//   delta_rule_kernel      four threads share a value channel, each with D / 4 key channels of it in registers; tokens
//                          in chunks, what does not depend on the state a chunk at a time (D = 32, 64, 128).
//   delta_rule_any_kernel  any D: the state in shared memory, a thread per value channel.
#include "common.cuh"

struct DeltaArgs {
  const float* proj;     // [T][ld]: columns r_off, k_off, v_off, a_off, g_off (each heads * D wide)
  long ld;
  int r_off, k_off, v_off, a_off, g_off;
  const float* w_raw;    // [T][ldw]
  long ldw;
  const void* w_bias;    // [heads * D]
  const void* a_bias;    // [heads * D]
  const void* norm_w;    // [heads * D]
  float* state;          // [slots][heads][D][D]
  const int* q_start;    // [R]
  const int* q_len;      // [R]
  const int* slot;       // [R]
  void* out;             // [T][heads * D]
  int heads, D;
  float decay_scale, unit_eps, eps;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

// Sum over the first `n` threads' values of a block of up to 256 threads, in a fixed order.
__device__ __forceinline__ float head_sum(float v, float* sh, int nwarps) {
  v = hb_warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nwarps; i++) t += sh[i];
  return t;
}

template <typename TW, typename TO>
__global__ void delta_rule_any_kernel(DeltaArgs A) {
  extern __shared__ float smem[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int D = A.D, h = blockIdx.x, req = blockIdx.y, j = threadIdx.x;
  const int nw = (blockDim.x + 31) >> 5;
  float* S = smem;                 // [D][D]
  float* vr = S + (size_t)D * D;   // r, w, au, k, u: [5][D]
  float* vw = vr + D, *vau = vw + D, *vk = vau + D, *vu = vk + D;
  float* sh = vu + D;              // [32]
  const bool on = j < D;
  float* Sg = A.state + ((size_t)A.slot[req] * A.heads + h) * D * D;
  if (on) for (int i = 0; i < D; i++) S[i * D + j] = Sg[i * D + j];
  const int t0 = A.q_start[req], n = A.q_len[req];
  const TW* wb = (const TW*)A.w_bias, *ab = (const TW*)A.a_bias, *nwt = (const TW*)A.norm_w;
  const int c = h * D + j;
  for (int t = t0; t < t0 + n; t++) {
    const float* row = A.proj + (size_t)t * A.ld;
    float kj = 0.f, vj = 0.f;
    if (on) {
      kj = row[A.k_off + c];
      vj = row[A.v_off + c];
    }
    const float kk = head_sum(kj * kj, sh, nw);     // (its first barrier also ends the token before)
    if (on) {
      const float uj = kj / sqrtf(kk + A.unit_eps);
      vr[j] = row[A.r_off + c];
      vw[j] = expf(-A.decay_scale * sigmoidf_(A.w_raw[(size_t)t * A.ldw + c] + hb_to_float(wb[c])));
      vau[j] = sigmoidf_(row[A.a_off + c] + hb_to_float(ab[c])) * uj;
      vk[j] = kj;
      vu[j] = uj;
    }
    __syncthreads();
    float o = 0.f;
    if (on) {
      float sa = 0.f;
      for (int i = 0; i < D; i++) sa = fmaf(vu[i], S[i * D + j], sa);
      for (int i = 0; i < D; i++) {
        const float s = fmaf(vk[i], vj, fmaf(vw[i], S[i * D + j], -vau[i] * sa));
        S[i * D + j] = s;
        o = fmaf(s, vr[i], o);
      }
    }
    const float oo = head_sum(o * o, sh, nw);
    if (on) {
      const float y = o * rsqrtf(oo / (float)D + A.eps) * hb_to_float(nwt[c]) * sigmoidf_(row[A.g_off + c]);
      ((TO*)A.out)[(size_t)t * A.heads * D + c] = hb_from_float<TO>(y);
    }
  }
  if (on) for (int i = 0; i < D; i++) Sg[i * D + j] = S[i * D + j];
}

// TPC threads per value channel, NR key channels each: D = TPC * NR, blockDim = D * TPC. Thread (q, j) holds
// S[q * NR + i][j], i < NR, in registers; the TPC parts of a sum over key channels meet in shared memory.
//
// The tokens go by in chunks of DR_CH. What does not depend on the state is done for a whole chunk at once, a warp per
// token: the unit key (one warp sum), decay and removal rate (expf), into shared memory; the raw values of the NEXT
// chunk are already on their way from global memory while the state walks through this one. The walk itself then
// costs, per token, 4 NR fused multiply-adds a thread, broadcast reads of the token's vectors and ONE barrier (for
// u^T S, whose parts must meet before the state moves; the parts of the output meet after the chunk). The head norm
// and the gate of the chunk's outputs are again a warp per token.
constexpr int DR_CH = 16;

template <typename TW, typename TO, int NR, int TPC>
__global__ void __launch_bounds__(NR * TPC * TPC, (NR * TPC * TPC <= 256 ? 2 : 1)) delta_rule_kernel(DeltaArgs A) {
  constexpr int D = NR * TPC, NT = D * TPC, NW = NT / 32, TPW = DR_CH / NW, CPL = D / 32;
  static_assert(TPW >= 1 && TPW * NW == DR_CH && CPL >= 1 && NR % 4 == 0, "chunk, warps and head size must fit");
  extern __shared__ __align__(16) float dr_smem[];
  float* vr = dr_smem;                 // [DR_CH][D] each
  float* vw = vr + DR_CH * D;
  float* vau = vw + DR_CH * D;
  float* vk = vau + DR_CH * D;
  float* vu = vk + DR_CH * D;
  float* vv = vu + DR_CH * D;
  float* vo = vv + DR_CH * D;          // [DR_CH][TPC][D]: the parts of a token's outputs, summed when the chunk is done
  float* xs = vo + DR_CH * TPC * D;    // [2][TPC][D]: the parts of u^T S of the token at hand (two buffers, one barrier a token)
  hb_pdl_launch();
  hb_pdl_wait();
  // a warp's lanes are 32 value channels j with the SAME part q of the key channels: what they read of the token's
  // vectors is one address for the whole warp (a broadcast, one pass through shared memory)
  const int h = blockIdx.x, req = blockIdx.y, tid = threadIdx.x, q = tid / D, j = tid % D, lane = tid & 31, warp = tid >> 5;
  float* Sg = A.state + ((size_t)A.slot[req] * A.heads + h) * D * D;
  float S[NR];
#pragma unroll
  for (int i = 0; i < NR; i++) S[i] = Sg[(q * NR + i) * D + j];
  const int t0 = A.q_start[req], n = A.q_len[req];
  const TW* wb = (const TW*)A.w_bias, *ab = (const TW*)A.a_bias, *nwt = (const TW*)A.norm_w;
  const int hc = h * D;

  // raw values of a chunk's tokens: warp `warp` takes tokens warp, warp + NW, ..; a lane channels lane, lane + 32, ..
  float pre[TPW][CPL][5];              // k, r, v, a_raw, w_raw
  float gate[TPW][CPL];                // the gate's raw values of the chunk being walked (asked for before the walk)
  float cab[CPL], cwb[CPL], cnw[CPL];  // this lane's channels of the two biases and the norm weight
#pragma unroll
  for (int y = 0; y < CPL; y++) {
    cab[y] = hb_to_float(ab[hc + lane + 32 * y]);
    cwb[y] = hb_to_float(wb[hc + lane + 32 * y]);
    cnw[y] = hb_to_float(nwt[hc + lane + 32 * y]);
  }
  auto fetch_gate = [&](int base) {
#pragma unroll
    for (int x = 0; x < TPW; x++) {
      const int tt = warp + x * NW;
      if (base + tt < n) {
        const float* row = A.proj + (size_t)(t0 + base + tt) * A.ld;
#pragma unroll
        for (int y = 0; y < CPL; y++) gate[x][y] = row[A.g_off + hc + lane + 32 * y];
      }
    }
  };
  auto fetch = [&](int base) {
#pragma unroll
    for (int x = 0; x < TPW; x++) {
      const int tt = warp + x * NW;
      if (base + tt < n) {
        const float* row = A.proj + (size_t)(t0 + base + tt) * A.ld;
        const float* wrow = A.w_raw + (size_t)(t0 + base + tt) * A.ldw;
#pragma unroll
        for (int y = 0; y < CPL; y++) {
          const int c = hc + lane + 32 * y;
          pre[x][y][0] = row[A.k_off + c];
          pre[x][y][1] = row[A.r_off + c];
          pre[x][y][2] = row[A.v_off + c];
          pre[x][y][3] = row[A.a_off + c];
          pre[x][y][4] = wrow[c];
        }
      }
    }
  };
  fetch(0);
  for (int base = 0; base < n; base += DR_CH) {
    // the chunk's vectors into shared memory
#pragma unroll
    for (int x = 0; x < TPW; x++) {
      const int tt = warp + x * NW;
      if (base + tt < n) {                                   // (uniform over the warp)
        float kk = 0.f;
#pragma unroll
        for (int y = 0; y < CPL; y++) kk = fmaf(pre[x][y][0], pre[x][y][0], kk);
        kk = hb_warp_sum(kk);
        const float inv = 1.f / sqrtf(kk + A.unit_eps);
#pragma unroll
        for (int y = 0; y < CPL; y++) {
          const int cl = lane + 32 * y;
          const float kj = pre[x][y][0], uj = kj * inv;
          vk[tt * D + cl] = kj;
          vu[tt * D + cl] = uj;
          vr[tt * D + cl] = pre[x][y][1];
          vv[tt * D + cl] = pre[x][y][2];
          vau[tt * D + cl] = sigmoidf_(pre[x][y][3] + cab[y]) * uj;
          vw[tt * D + cl] = expf(-A.decay_scale * sigmoidf_(pre[x][y][4] + cwb[y]));
        }
      }
    }
    __syncthreads();
    fetch_gate(base);                                        // both in flight during the walk
    if (base + DR_CH < n) fetch(base + DR_CH);
    const int m = min(DR_CH, n - base);
    for (int tt = 0; tt < m; tt++) {
      // (heads of up to 64) all of the token's vectors are asked for at once: one wait for shared memory a token
      constexpr bool HOIST = NR <= 16;
      const float4* up = (const float4*)(vu + tt * D + q * NR);
      const float4* kp = (const float4*)(vk + tt * D + q * NR);
      const float4* wp = (const float4*)(vw + tt * D + q * NR);
      const float4* ap = (const float4*)(vau + tt * D + q * NR);
      const float4* rp = (const float4*)(vr + tt * D + q * NR);
      float4 u[HOIST ? NR / 4 : 1], k[HOIST ? NR / 4 : 1], w[HOIST ? NR / 4 : 1], a[HOIST ? NR / 4 : 1], r[HOIST ? NR / 4 : 1];
      if (HOIST) {
#pragma unroll
        for (int i = 0; i < NR / 4; i++) { u[i] = up[i]; k[i] = kp[i]; w[i] = wp[i]; a[i] = ap[i]; r[i] = rp[i]; }
      }
      const float vj = vv[tt * D + j];
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int i = 0; i < NR / 4; i++) {
        const float4 uu = HOIST ? u[i] : up[i];
        s0 = fmaf(uu.x, S[4 * i], s0); s1 = fmaf(uu.y, S[4 * i + 1], s1);
        s2 = fmaf(uu.z, S[4 * i + 2], s2); s3 = fmaf(uu.w, S[4 * i + 3], s3);
      }
      float* x = xs + (tt & 1) * TPC * D;
      x[q * D + j] = (s0 + s1) + (s2 + s3);
      __syncthreads();
      float sa = x[j];
#pragma unroll
      for (int qq = 1; qq < TPC; qq++) sa += x[qq * D + j];
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < NR / 4; i++) {
        const float4 kk = HOIST ? k[i] : kp[i], ww = HOIST ? w[i] : wp[i], aa = HOIST ? a[i] : ap[i], rr = HOIST ? r[i] : rp[i];
        S[4 * i] = fmaf(kk.x, vj, fmaf(ww.x, S[4 * i], -aa.x * sa));             o0 = fmaf(S[4 * i], rr.x, o0);
        S[4 * i + 1] = fmaf(kk.y, vj, fmaf(ww.y, S[4 * i + 1], -aa.y * sa));     o1 = fmaf(S[4 * i + 1], rr.y, o1);
        S[4 * i + 2] = fmaf(kk.z, vj, fmaf(ww.z, S[4 * i + 2], -aa.z * sa));     o2 = fmaf(S[4 * i + 2], rr.z, o2);
        S[4 * i + 3] = fmaf(kk.w, vj, fmaf(ww.w, S[4 * i + 3], -aa.w * sa));     o3 = fmaf(S[4 * i + 3], rr.w, o3);
      }
      vo[(tt * TPC + q) * D + j] = (o0 + o1) + (o2 + o3);
    }
    __syncthreads();
    // the chunk's outputs: head norm, weight and gate, a warp per token
#pragma unroll
    for (int x = 0; x < TPW; x++) {
      const int tt = warp + x * NW;
      if (base + tt < n) {
        float ov[CPL], oo = 0.f;
#pragma unroll
        for (int y = 0; y < CPL; y++) {
          ov[y] = vo[tt * TPC * D + lane + 32 * y];
#pragma unroll
          for (int qq = 1; qq < TPC; qq++) ov[y] += vo[(tt * TPC + qq) * D + lane + 32 * y];
          oo = fmaf(ov[y], ov[y], oo);
        }
        oo = hb_warp_sum(oo);
        const float f = rsqrtf(oo / (float)D + A.eps);
        const size_t t = (size_t)(t0 + base + tt);
#pragma unroll
        for (int y = 0; y < CPL; y++) {
          const int c = hc + lane + 32 * y;
          ((TO*)A.out)[t * A.heads * D + c] = hb_from_float<TO>(ov[y] * f * cnw[y] * sigmoidf_(gate[x][y]));
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NR; i++) Sg[(q * NR + i) * D + j] = S[i];
}

template <typename TW, typename TO, int NR, int TPC>
static int delta_rule_launch_reg(const DeltaArgs& A, dim3 grid, cudaStream_t s) {
  constexpr int D = NR * TPC;
  const size_t smem = ((size_t)(6 + TPC) * DR_CH * D + 2 * TPC * D) * sizeof(float);
  auto kern = delta_rule_kernel<TW, TO, NR, TPC>;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) HB_FAIL("hb_delta_rule: %s", cudaGetErrorString(e));
    configured = true;
  }
  hb_launch(kern, grid, D * TPC, smem, s, A);
  return 0;
}

template <typename TW, typename TO>
static int delta_rule_launch(const DeltaArgs& A, int R, cudaStream_t s) {
  const dim3 grid(A.heads, R);
  switch (A.D) {
    case 32: return delta_rule_launch_reg<TW, TO, 8, 4>(A, grid, s);
    case 64: return delta_rule_launch_reg<TW, TO, 16, 4>(A, grid, s);
    case 128: return delta_rule_launch_reg<TW, TO, 32, 4>(A, grid, s);
    default: break;
  }
  const int threads = (A.D + 31) / 32 * 32;
  const size_t smem = ((size_t)A.D * A.D + 5 * (size_t)A.D + 32) * sizeof(float);
  if (threads > 1024 || smem > 200 * 1024) HB_FAIL("hb_delta_rule: heads of %d are too wide for one block's shared memory", A.D);
  auto kern = delta_rule_any_kernel<TW, TO>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) HB_FAIL("hb_delta_rule: %s", cudaGetErrorString(e));
  }
  hb_launch(kern, grid, threads, smem, s, A);
  return 0;
}

// force_any: run the shared-memory kernel also where a register kernel exists (tests compare the two).
HB_EXPORT int hb_delta_rule(const float* proj, long ld, int r_off, int k_off, int v_off, int a_off, int g_off,
                            const float* w_raw, long ldw, const void* w_bias, const void* a_bias, const void* norm_w,
                            int w_dt, float* state, const int* q_start, const int* q_len, const int* slot, void* out,
                            int out_dt, int R, int heads, int D, float decay_scale, float unit_eps, float eps,
                            int force_any, cudaStream_t s) {
  if (R <= 0) return 0;
  if (heads <= 0 || D <= 0) HB_FAIL("hb_delta_rule: %d heads of %d", heads, D);
  if (R > 65535) HB_FAIL("hb_delta_rule: %d requests are beyond the grid limit", R);
  DeltaArgs A{proj, ld, r_off, k_off, v_off, a_off, g_off, w_raw, ldw, w_bias, a_bias, norm_w, state, q_start, q_len, slot,
              out, heads, D, decay_scale, unit_eps, eps};
  int r = -1;
  HB_DISPATCH_2(w_dt, out_dt, "hb_delta_rule", {
    if (force_any) {
      const int threads = (D + 31) / 32 * 32;
      const size_t smem = ((size_t)D * D + 5 * (size_t)D + 32) * sizeof(float);
      if (threads > 1024 || smem > 200 * 1024) HB_FAIL("hb_delta_rule: heads of %d are too wide for one block's shared memory", D);
      auto kern = delta_rule_any_kernel<TA, TB>;
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) HB_FAIL("hb_delta_rule: %s", cudaGetErrorString(e));
      }
      hb_launch(kern, dim3(heads, R), threads, smem, s, A);
      r = 0;
    } else {
      r = delta_rule_launch<TA, TB>(A, R, s);
    }
  });
  if (r) return r;
  HB_CHECK_LAUNCH("hb_delta_rule");
  return 0;
}
