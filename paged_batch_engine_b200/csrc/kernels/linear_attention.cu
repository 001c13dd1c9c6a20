// Linear attention with a fixed decay per head, as a recurrence over a float32 state:
//   S_t = lambda_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t      (S: [D, E] per head and request)
// q, k (D wide) and v (E wide) are slices of one wider projection matrix; an activation (silu)
// and a scale on k are applied as they are read, in float32.  The state lives in a row of a
// per-request table, is read at the start of a request's rows of this step and written back
// at their end; the step function zeroes it before a request's first tokens.
//
// One warp per (request, head, slice of value columns).  A lane owns one value column e and
// holds S[:, e] in registers (or, for D beyond 128, PARTS lanes share a column and each holds
// D / PARTS of it); per token the warp stages q_t and k_t in shared memory, every lane updates
// its column and takes its dot product with q_t.  The next token's q, k and v are fetched
// while the current one is computed.  Prompt portions and single decoded tokens take the same
// path: a request brings q_len rows.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
struct LinAttnParams {
  const void* q;            // element (row 0, head 0, 0) of q inside the projection
  const void* k;
  const void* v;
  int ld;                   // row stride of the projection, elements
  float* out;               // [T, H * E]
  float* state;             // [slots, H, D, E]
  const float* decay;       // [H]
  const int32_t* q_start;   // [R]
  const int32_t* q_len;     // [R]
  const int32_t* slots;     // [R] state row of each request
  int H, D, E;
  float k_scale;
  int act;                  // 1: silu on q, k and v
};

__device__ __forceinline__ float act_of(float x, int act) { return act ? x / (1.0f + expf(-x)) : x; }

// DPT: state elements a lane holds (its share of D); PARTS lanes share one value column
template <typename T, int DPT, int PARTS>
__global__ void __launch_bounds__(32) linear_attention_kernel(LinAttnParams p) {
  constexpr int COLS = 32 / PARTS;             // value columns a warp covers
  constexpr int DMAX = DPT * PARTS;
  __shared__ __align__(16) float qs[DMAX], ks[DMAX];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x;
  const int part = lane % PARTS, col = lane / PARTS;
  const int e = blockIdx.z * COLS + col;
  const int D = p.D, E = p.E, H = p.H;
  const int n = p.q_len[r];
  if (n <= 0) return;
  const int t0 = p.q_start[r];
  const bool live = e < E;
  const int d0 = part * DPT;                   // this lane's first state row
  float* st = p.state + (((size_t)p.slots[r] * H + h) * D) * E;
  float S[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = (live && d0 + i < D) ? st[(size_t)(d0 + i) * E + e] : 0.f;
  const float lam = p.decay[h];
  const T* qp = (const T*)p.q + (size_t)h * D;
  const T* kp = (const T*)p.k + (size_t)h * D;
  const T* vp = (const T*)p.v + (size_t)h * E;
  constexpr int PER = (DMAX + 31) / 32;        // q and k elements a lane fetches per token
  float qn[PER], kn[PER], vn;
  auto fetch = [&](int t) {
    const size_t row = (size_t)(t0 + t) * p.ld;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + i * 32;
      qn[i] = d < D ? act_of(to_float(qp[row + d]), p.act) : 0.f;
      kn[i] = d < D ? act_of(to_float(kp[row + d]), p.act) * p.k_scale : 0.f;
    }
    vn = live ? act_of(to_float(vp[row + e]), p.act) : 0.f;
  };
  fetch(0);
  for (int t = 0; t < n; ++t) {
    __syncwarp();
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + i * 32;
      if (d < DMAX) {
        qs[d] = qn[i];
        ks[d] = kn[i];
      }
    }
    const float v = vn;
    __syncwarp();
    if (t + 1 < n) fetch(t + 1);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(ks + d0 + i);
      const float4 q4 = *reinterpret_cast<const float4*>(qs + d0 + i);
      S[i] = fmaf(lam, S[i], k4.x * v);
      o = fmaf(S[i], q4.x, o);
      S[i + 1] = fmaf(lam, S[i + 1], k4.y * v);
      o = fmaf(S[i + 1], q4.y, o);
      S[i + 2] = fmaf(lam, S[i + 2], k4.z * v);
      o = fmaf(S[i + 2], q4.z, o);
      S[i + 3] = fmaf(lam, S[i + 3], k4.w * v);
      o = fmaf(S[i + 3], q4.w, o);
    }
#pragma unroll
    for (int m = 1; m < PARTS; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
    if (live && part == 0) p.out[(size_t)(t0 + t) * H * E + (size_t)h * E + e] = o;
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < D) st[(size_t)(d0 + i) * E + e] = S[i];
  }
}

template <typename T, int DPT, int PARTS>
void launch_la(const LinAttnParams& p, int R, cudaStream_t stream) {
  constexpr int COLS = 32 / PARTS;
  dim3 grid(R, p.H, (p.E + COLS - 1) / COLS);
  launch_k(linear_attention_kernel<T, DPT, PARTS>, grid, 32, 0, stream, p);
}

template <typename T>
int dispatch_la(const LinAttnParams& p, int R, cudaStream_t stream) {
  const int D = p.D;
  if (D <= 16) launch_la<T, 16, 1>(p, R, stream);
  else if (D <= 32) launch_la<T, 32, 1>(p, R, stream);
  else if (D <= 64) launch_la<T, 64, 1>(p, R, stream);
  else if (D <= 128) launch_la<T, 128, 1>(p, R, stream);
  else if (D <= 256) launch_la<T, 128, 2>(p, R, stream);
  else if (D <= 512) launch_la<T, 128, 4>(p, R, stream);
  else return (int)cudaErrorInvalidValue;
  return launch_status();
}
}  // namespace

PBE_EXPORT int pbe_linear_attention(const void* q, const void* k, const void* v, int ld, int dtype, float* out,
                                    float* state, const float* decay, const int32_t* q_start, const int32_t* q_len,
                                    const int32_t* slots, int R, int H, int D, int E, float k_scale, int act,
                                    cudaStream_t stream) {
  if (R <= 0) return 0;
  LinAttnParams p{q, k, v, ld, out, state, decay, q_start, q_len, slots, H, D, E, k_scale, act};
  return dtype == PBE_F32 ? dispatch_la<float>(p, R, stream) : dispatch_la<__nv_bfloat16>(p, R, stream);
}
