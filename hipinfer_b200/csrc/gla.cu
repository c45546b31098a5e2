// Gated linear attention: a linear recurrence with one state matrix per head and a decay per key channel.
//
// For each head, with a state S [D][E] (key channel by value channel) that starts at zero and is carried from token to
// token in 32-bit:
//     alpha = sigmoid(z + b)^(1 / tau)               per key channel; computed as exp(log_sigmoid(z + b) / tau)
//     S <- diag(alpha) S + k v^T                     the decay acts on the rows of S (key channels)
//     o = S^T (q / sqrt(D))
// then o is divided by its root mean square over E (eps inside the root), multiplied by a weight vector over E (shared
// by the heads) and by silu(g), and rounded once. q, k, v, g are columns of one 32-bit projection result, z of another.
//
// A block owns (head, request) and walks the request's rows of the step in order, from and into its state slot. The
// state lives in registers: KS threads share a value channel, each holding every KS-th key channel (at most DPT of
// them). Tokens go by in chunks of GL_CH: a chunk's raw rows are asked for a chunk ahead (cp.async into shared memory),
// what does not depend on the state (decays, the scaled query) is prepared there in place, the walk reads it by
// broadcast and writes the raw o, and the head norm, weight and gate follow a warp a token. A token's arithmetic does not depend on where a chunk or a portion starts. Requests,
// lengths and state slots are read from device arrays, so a decode step can be replayed from a CUDA graph.
#include "common.cuh"

constexpr int GL_CH = 16;

struct GlaArgs {
  const float* proj; long ld; int q_off, k_off, v_off, g_off;
  const float* z; long ldz;
  const void* a_bias; const void* norm_w;       // [H * D], [E]
  float* state;                                 // [slots][H][D][E]
  const int* q_start; const int* q_len; const int* slot;
  void* out;                                    // [T][H * E]
  int H, D, E, KS, vec4;
  float inv_tau, eps, q_scale;
};

// threads a block may have so that DPT state values (and what goes with them) stay in registers
template <int DPT> struct GlaThreads { static constexpr int MAX = DPT <= 8 ? 1024 : DPT <= 32 ? 512 : 256; };

__device__ __forceinline__ void gl_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void gl_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// FAST: D == DPT * KS and D, E multiples of 4 with 16-byte aligned rows. A thread then holds the DPT CONTIGUOUS key channels
// ks * DPT .. of its value channel and reads their decays, keys and queries four at a time (the per-channel vectors lie in
// shared memory with 4 floats of padding after every DPT, so that the KS slices fall on different banks); no bounds are
// checked and every offset is a constant. Otherwise (any sizes) a thread holds every KS-th key channel.
template <int DPT, bool FAST, typename TW, typename TO>
__global__ void __launch_bounds__(GlaThreads<DPT>::MAX, 1) gla_kernel(GlaArgs A) {
  extern __shared__ __align__(16) float gsm[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int D = A.D, E = A.E, KS = A.KS, H = A.H;
  const int e = tid / KS, ks = tid - e * KS;
  const bool live = e < E;
  const int t0 = A.q_start[r], len = A.q_len[r];
  float* S_g = A.state + ((size_t)A.slot[r] * H + h) * D * E;
  // a chunk's rows in shared memory, two chunks deep: per token [q (D) | k (D) | z -> alpha (D) | v (E) | g (E)]
  const int DQ = FAST ? D + 4 * KS : D;            // a per-channel vector with its padding
  const int RW = 3 * DQ + 2 * E;
  auto pidx = [&](int d) { return FAST ? d + (d / DPT) * 4 : d; };
  float* stage0 = gsm;                          // [2][GL_CH][RW]
  float* oc = gsm + 2 * GL_CH * RW;             // [GL_CH][E]
  float S[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = FAST ? ks * DPT + i : i * KS + ks;
    S[i] = (live && d < D) ? S_g[(size_t)d * E + e] : 0.f;
  }
  const TW* ab = (const TW*)A.a_bias + (size_t)h * D;
  const TW* nw = (const TW*)A.norm_w;
  // the raw rows of a chunk are asked for a chunk ahead (cp.async), so that the walk never waits for memory
  auto fetch = [&](int buf, int c0) {
    const int n = min(GL_CH, len - c0);
    float* st = stage0 + buf * GL_CH * RW;
    if (A.vec4) {
      const int cd = D >> 2, ce = E >> 2, per = 3 * cd + 2 * ce;
      for (int i = tid; i < n * per; i += nthr) {
        const int j = i / per, c = i - j * per;
        const size_t t = (size_t)(t0 + c0 + j);
        const float* src;
        int dst;
        if (c < cd) { src = A.proj + t * A.ld + A.q_off + h * D + 4 * c; dst = pidx(4 * c); }
        else if (c < 2 * cd) { src = A.proj + t * A.ld + A.k_off + h * D + 4 * (c - cd); dst = DQ + pidx(4 * (c - cd)); }
        else if (c < 3 * cd) { src = A.z + t * A.ldz + h * D + 4 * (c - 2 * cd); dst = 2 * DQ + pidx(4 * (c - 2 * cd)); }
        else if (c < 3 * cd + ce) { src = A.proj + t * A.ld + A.v_off + h * E + 4 * (c - 3 * cd); dst = 3 * DQ + 4 * (c - 3 * cd); }
        else { src = A.proj + t * A.ld + A.g_off + h * E + 4 * (c - 3 * cd - ce); dst = 3 * DQ + E + 4 * (c - 3 * cd - ce); }
        gl_cp16(st + j * RW + dst, src);
      }
    } else {
      for (int i = tid; i < n * RW; i += nthr) {
        const int j = i / RW, c = i - j * RW;
        const size_t t = (size_t)(t0 + c0 + j);
        const float* src;
        if (c < D) src = A.proj + t * A.ld + A.q_off + h * D + c;
        else if (c < 2 * D) src = A.proj + t * A.ld + A.k_off + h * D + (c - D);
        else if (c < 3 * D) src = A.z + t * A.ldz + h * D + (c - 2 * D);
        else if (c < 3 * D + E) src = A.proj + t * A.ld + A.v_off + h * E + (c - 3 * D);
        else src = A.proj + t * A.ld + A.g_off + h * E + (c - 3 * D - E);
        gl_cp4(st + j * RW + c, src);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (len > 0) fetch(0, 0);
  int buf = 0;
  for (int c0 = 0; c0 < len; c0 += GL_CH, buf ^= 1) {
    const int n = min(GL_CH, len - c0);
    if (c0 + GL_CH < len) {
      fetch(buf ^ 1, c0 + GL_CH);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    float* st = stage0 + buf * GL_CH * RW;
    // what does not depend on the state: the scaled query and the decay, in place
    for (int i = tid; i < n * D; i += nthr) {
      const int j = i / D, d = i - j * D;
      float* row = st + j * RW;
      const int pd = pidx(d);
      row[pd] *= A.q_scale;
      const float zz = row[2 * DQ + pd] + hb_to_float(ab[d]);
      // log sigmoid(z) = -(max(-z, 0) + log1p(exp(-|z|)))
      const float ls = -(fmaxf(-zz, 0.f) + log1pf(expf(-fabsf(zz))));
      row[2 * DQ + pd] = expf(ls * A.inv_tau);
    }
    __syncthreads();
    for (int j = 0; j < n; j++) {
      const float* row = st + j * RW;
      const float v = live ? row[3 * DQ + e] : 0.f;
      const float* qj = row;
      const float* kj = row + DQ;
      const float* aj = row + 2 * DQ;
      float o = 0.f;
      if constexpr (FAST) {
        const int sb = ks * (DPT + 4);
        float o2 = 0.f;                        // two chains: the sum over a thread's channels is half as deep
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 a4 = *(const float4*)(aj + sb + i), k4 = *(const float4*)(kj + sb + i), q4 = *(const float4*)(qj + sb + i);
          S[i] = fmaf(a4.x, S[i], k4.x * v);
          S[i + 1] = fmaf(a4.y, S[i + 1], k4.y * v);
          S[i + 2] = fmaf(a4.z, S[i + 2], k4.z * v);
          S[i + 3] = fmaf(a4.w, S[i + 3], k4.w * v);
          o = fmaf(S[i], q4.x, o);
          o2 = fmaf(S[i + 1], q4.y, o2);
          o = fmaf(S[i + 2], q4.z, o);
          o2 = fmaf(S[i + 3], q4.w, o2);
        }
        o += o2;
      } else {
#pragma unroll
        for (int i = 0; i < DPT; i++) {
          const int d = i * KS + ks;
          if (d < D) {
            S[i] = fmaf(aj[d], S[i], kj[d] * v);
            o = fmaf(S[i], qj[d], o);
          }
        }
      }
      for (int m = 1; m < KS; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (live && ks == 0) oc[j * E + e] = o;
    }
    __syncthreads();
    for (int j = warp; j < n; j += nthr >> 5) {
      float ss = 0.f;
      for (int ee = lane; ee < E; ee += 32) ss = fmaf(oc[j * E + ee], oc[j * E + ee], ss);
      const float f = rsqrtf(hb_warp_sum(ss) / (float)E + A.eps);
      const size_t t = (size_t)(t0 + c0 + j);
      const float* grow = st + j * RW + 3 * DQ + E;
      for (int ee = lane; ee < E; ee += 32) {
        const float g = grow[ee];
        const float y = oc[j * E + ee] * f * hb_to_float(nw[ee]) * (g / (1.f + expf(-g)));
        ((TO*)A.out)[t * (size_t)(H * E) + h * E + ee] = hb_from_float<TO>(y);
      }
    }
    __syncthreads();             // the buffer is free for the chunk after the next
  }
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = FAST ? ks * DPT + i : i * KS + ks;
    if (live && d < D) S_g[(size_t)d * E + e] = S[i];
  }
}

HB_EXPORT int hb_gla(const float* proj, long ld, int q_off, int k_off, int v_off, int g_off, const float* z, long ldz,
                     const void* a_bias, const void* norm_w, int w_dt, float* state, const int* q_start, const int* q_len,
                     const int* slot, void* out, int o_dt, int n_requests, int H, int D, int E, float tau, float eps,
                     cudaStream_t s) {
  if (n_requests <= 0) return 0;
  if (E > 1024) HB_FAIL("hb_gla: values of %d are too wide", E);
  // threads a value channel (a power of two up to 32): the fewest that give the block 256 threads, else the most that
  // fit; a thread holds ceil(D / ks) key channels of its value channel, which bounds the block's threads
  int ks = 0;
  for (int c = 1; c <= 32; c *= 2) {
    const int per_c = (D + c - 1) / c, threads_c = ((E * c + 31) / 32) * 32;
    if (per_c > 64) continue;
    const int limit = per_c <= 8 ? 1024 : per_c <= 32 ? 512 : 256;
    if (threads_c > limit) break;
    ks = c;
    if (threads_c >= 256) break;
  }
  if (!ks) HB_FAIL("hb_gla: heads of %d x %d do not fit a block's registers", D, E);
  const int per = (D + ks - 1) / ks;
  GlaArgs A;
  A.proj = proj; A.ld = ld; A.q_off = q_off; A.k_off = k_off; A.v_off = v_off; A.g_off = g_off; A.z = z; A.ldz = ldz;
  A.a_bias = a_bias; A.norm_w = norm_w; A.state = state; A.q_start = q_start; A.q_len = q_len; A.slot = slot; A.out = out;
  A.H = H; A.D = D; A.E = E; A.KS = ks; A.inv_tau = 1.f / tau; A.eps = eps; A.q_scale = 1.f / sqrtf((float)D);
  const int threads = ((E * ks + 31) / 32) * 32;
  // whole 16-byte copies where every row segment starts on a 16-byte boundary
  A.vec4 = !((D | E | q_off | k_off | v_off | g_off) & 3) && !((ld | ldz) & 3) && !(((uintptr_t)proj | (uintptr_t)z) & 15);
  const bool fast = A.vec4 && per * ks == D && (per == 8 || per == 16 || per == 32 || per == 64);
  const int DQ = fast ? D + 4 * ks : D;
  const size_t smem = (size_t)(2 * GL_CH * (3 * DQ + 2 * E) + GL_CH * E) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_gla: heads of %d x %d do not fit shared memory", D, E);
  dim3 grid(H, n_requests);
#define GL_LAUNCH(DPT)                                                                                               \
  HB_DISPATCH_2(w_dt, o_dt, "hb_gla", do {                                                                           \
    if (fast) {                                                                                                      \
      auto kern = gla_kernel<DPT, true, TA, TB>;                                                                     \
      if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
      hb_launch(kern, grid, dim3(threads), smem, s, A);                                                              \
    } else {                                                                                                         \
      auto kern = gla_kernel<DPT, false, TA, TB>;                                                                    \
      if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
      hb_launch(kern, grid, dim3(threads), smem, s, A);                                                              \
    }                                                                                                                \
  } while (0))
  if (per <= 8) GL_LAUNCH(8);
  else if (per <= 16) GL_LAUNCH(16);
  else if (per <= 32) GL_LAUNCH(32);
  else GL_LAUNCH(64);
#undef GL_LAUNCH
  HB_CHECK_LAUNCH("hb_gla");
  return 0;
}
