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
// them). Tokens go by in chunks of GL_CH: what does not depend on the state (decays, the scaled query) is prepared a
// chunk at a time in shared memory, the walk reads it by broadcast and writes the raw o, and the head norm, weight and
// gate follow a warp a token. A token's arithmetic does not depend on where a chunk or a portion starts. Requests,
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
  int H, D, E, KS;
  float inv_tau, eps, q_scale;
};

// threads a block may have so that DPT state values (and what goes with them) stay in registers
template <int DPT> struct GlaThreads { static constexpr int MAX = DPT <= 8 ? 1024 : DPT <= 32 ? 512 : 256; };

template <int DPT, typename TW, typename TO>
__global__ void __launch_bounds__(GlaThreads<DPT>::MAX, 1) gla_kernel(GlaArgs A) {
  extern __shared__ float gsm[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int D = A.D, E = A.E, KS = A.KS, H = A.H;
  const int e = tid / KS, ks = tid - e * KS;
  const bool live = e < E;
  const int t0 = A.q_start[r], len = A.q_len[r];
  float* S_g = A.state + ((size_t)A.slot[r] * H + h) * D * E;
  float* qs = gsm;                 // [GL_CH][D]
  float* kk = qs + GL_CH * D;      // [GL_CH][D]
  float* al = kk + GL_CH * D;      // [GL_CH][D]
  float* vv = al + GL_CH * D;      // [GL_CH][E]
  float* oc = vv + GL_CH * E;      // [GL_CH][E]
  float S[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = i * KS + ks;
    S[i] = (live && d < D) ? S_g[(size_t)d * E + e] : 0.f;
  }
  const TW* ab = (const TW*)A.a_bias + (size_t)h * D;
  const TW* nw = (const TW*)A.norm_w;
  for (int c0 = 0; c0 < len; c0 += GL_CH) {
    const int n = min(GL_CH, len - c0);
    __syncthreads();             // the chunk before is done with the buffers
    for (int i = tid; i < n * D; i += nthr) {
      const int j = i / D, d = i - j * D;
      const float* row = A.proj + (size_t)(t0 + c0 + j) * A.ld;
      qs[i] = row[A.q_off + h * D + d] * A.q_scale;
      kk[i] = row[A.k_off + h * D + d];
      const float zz = A.z[(size_t)(t0 + c0 + j) * A.ldz + h * D + d] + hb_to_float(ab[d]);
      // log sigmoid(z) = -(max(-z, 0) + log1p(exp(-|z|)))
      const float ls = -(fmaxf(-zz, 0.f) + log1pf(expf(-fabsf(zz))));
      al[i] = expf(ls * A.inv_tau);
    }
    for (int i = tid; i < n * E; i += nthr) {
      const int j = i / E, ee = i - j * E;
      vv[i] = A.proj[(size_t)(t0 + c0 + j) * A.ld + A.v_off + h * E + ee];
    }
    __syncthreads();
    for (int j = 0; j < n; j++) {
      const float v = live ? vv[j * E + e] : 0.f;
      const float* qj = qs + j * D;
      const float* kj = kk + j * D;
      const float* aj = al + j * D;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; i++) {
        const int d = i * KS + ks;
        if (d < D) {
          S[i] = fmaf(aj[d], S[i], kj[d] * v);
          o = fmaf(S[i], qj[d], o);
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
      for (int ee = lane; ee < E; ee += 32) {
        const float g = A.proj[t * A.ld + A.g_off + h * E + ee];
        const float y = oc[j * E + ee] * f * hb_to_float(nw[ee]) * (g / (1.f + expf(-g)));
        ((TO*)A.out)[t * (size_t)(H * E) + h * E + ee] = hb_from_float<TO>(y);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = i * KS + ks;
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
  const size_t smem = (size_t)GL_CH * (3 * D + 2 * E) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_gla: heads of %d x %d do not fit shared memory", D, E);
  dim3 grid(H, n_requests);
#define GL_LAUNCH(DPT)                                                                                               \
  HB_DISPATCH_2(w_dt, o_dt, "hb_gla", do {                                                                           \
    auto kern = gla_kernel<DPT, TA, TB>;                                                                             \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
    hb_launch(kern, grid, dim3(threads), smem, s, A);                                                                \
  } while (0))
  if (per <= 8) GL_LAUNCH(8);
  else if (per <= 16) GL_LAUNCH(16);
  else if (per <= 32) GL_LAUNCH(32);
  else GL_LAUNCH(64);
#undef GL_LAUNCH
  HB_CHECK_LAUNCH("hb_gla");
  return 0;
}
