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
//   delta_rule_kernel      TPC threads share a value channel, each with NR = D / TPC key channels of it in registers;
//                          the two sums over key channels end with shuffles among the TPC threads (D = 32, 64, 128).
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

// TPC threads per value channel, NR key channels each: D = TPC * NR, blockDim = D * TPC (lanes of a channel are
// neighbours, so the shuffles stay inside a warp). Thread (j, q) holds S[q * NR + i][j], i < NR.
template <typename TW, typename TO, int NR, int TPC>
__global__ void __launch_bounds__(NR * TPC * TPC) delta_rule_kernel(DeltaArgs A) {
  constexpr int D = NR * TPC, NT = D * TPC, NW = NT / 32;
  __shared__ float vr[D], vw[D], vau[D], vk[D], vu[D], sh[32];
  hb_pdl_launch();
  hb_pdl_wait();
  const int h = blockIdx.x, req = blockIdx.y, tid = threadIdx.x, j = tid / TPC, q = tid % TPC;
  float* Sg = A.state + ((size_t)A.slot[req] * A.heads + h) * D * D;
  float S[NR];
#pragma unroll
  for (int i = 0; i < NR; i++) S[i] = Sg[(q * NR + i) * D + j];
  const int t0 = A.q_start[req], n = A.q_len[req];
  const TW* wb = (const TW*)A.w_bias, *ab = (const TW*)A.a_bias, *nwt = (const TW*)A.norm_w;
  const int c = h * D + j;
  for (int t = t0; t < t0 + n; t++) {
    const float* row = A.proj + (size_t)t * A.ld;
    // the first D threads prepare channel `tid` of the token's vectors
    const int cc = h * D + tid;
    float kj = 0.f;
    if (tid < D) kj = row[A.k_off + cc];
    const float kk = head_sum(kj * kj, sh, NW);
    if (tid < D) {
      const float uj = kj / sqrtf(kk + A.unit_eps);
      vr[tid] = row[A.r_off + cc];
      vw[tid] = expf(-A.decay_scale * sigmoidf_(A.w_raw[(size_t)t * A.ldw + cc] + hb_to_float(wb[cc])));
      vau[tid] = sigmoidf_(row[A.a_off + cc] + hb_to_float(ab[cc])) * uj;
      vk[tid] = kj;
      vu[tid] = uj;
    }
    const float vj = row[A.v_off + c];
    __syncthreads();
    float sa = 0.f;
#pragma unroll
    for (int i = 0; i < NR; i++) sa = fmaf(vu[q * NR + i], S[i], sa);
#pragma unroll
    for (int o_ = 1; o_ < TPC; o_ <<= 1) sa += __shfl_xor_sync(0xffffffffu, sa, o_);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < NR; i++) {
      const int ki = q * NR + i;
      S[i] = fmaf(vk[ki], vj, fmaf(vw[ki], S[i], -vau[ki] * sa));
      o = fmaf(S[i], vr[ki], o);
    }
#pragma unroll
    for (int o_ = 1; o_ < TPC; o_ <<= 1) o += __shfl_xor_sync(0xffffffffu, o, o_);
    const float oo = head_sum(q == 0 ? o * o : 0.f, sh, NW);
    if (q == 0) {
      const float y = o * rsqrtf(oo / (float)D + A.eps) * hb_to_float(nwt[c]) * sigmoidf_(row[A.g_off + c]);
      ((TO*)A.out)[(size_t)t * A.heads * D + c] = hb_from_float<TO>(y);
    }
  }
#pragma unroll
  for (int i = 0; i < NR; i++) Sg[(q * NR + i) * D + j] = S[i];
}

template <typename TW, typename TO>
static int delta_rule_launch(const DeltaArgs& A, int R, cudaStream_t s) {
  const dim3 grid(A.heads, R);
  switch (A.D) {
    case 32: hb_launch(delta_rule_kernel<TW, TO, 8, 4>, grid, 128, 0, s, A); return 0;
    case 64: hb_launch(delta_rule_kernel<TW, TO, 16, 4>, grid, 256, 0, s, A); return 0;
    case 128: hb_launch(delta_rule_kernel<TW, TO, 16, 8>, grid, 1024, 0, s, A); return 0;
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
