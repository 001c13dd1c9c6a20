// Linear attention with a decay per head, as a recurrence over a float32 state:
//   S_t = lambda_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t      (S: [D, E] per head and request)
// and its selective form, in which the decay and a factor on v differ from token to token, q and
// k are shared by a group of heads and the output has a skip term:
//   S_t = a_{t,h} S_{t-1} + k_t (s_{t,h} v_t)^T,   o_t = S_t^T q_t + skip_h v_t
// q, k (D wide) and v (E wide) are slices of one wider projection matrix; an activation (silu)
// and a scale on k are applied as they are read, in float32.  The state lives in a row of a
// per-request table, is read at the start of a request's rows of this step and written back
// at their end; the step function zeroes it before a request's first tokens.
//
// One block per (request, head, slice of value columns).  A thread owns (a share of) one value
// column e and holds S[:, e] in registers: all of it for D up to 32, else PARTS neighbouring
// lanes hold D / PARTS elements each; the block stages q and k of a batch of tokens in shared
// memory (two buffers, one barrier a batch; a batch's loads are all in flight at once and the batch
// after next is fetched while the current one is computed), every thread updates its share token
// by token and takes its part of the dot product with q_t, and the parts are added by shuffles.  Prompt portions and single decoded tokens take the same
// path: a request brings q_len rows.
//
// Long prompt portions are cut into chunks that run side by side (the launcher's work items):
// first every chunk but a request's last runs from a zero state and leaves only its own
// contribution U_c = sum_j lambda^(n_c-1-j) k_j v_j^T in scratch memory; a scan then turns these
// into the states at the chunks' starts, S_c = lambda^(n_{c-1}) S_{c-1} + U_{c-1}, beginning with
// the request's state row; last, every chunk runs again from its start state and writes its
// outputs, the request's last chunk leaving the new state in the row.  The arithmetic per token
// is the recurrence's own, so a cut changes a result by the rounding of float32 sums only.
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
  // work items instead of requests when not null: [n, 4] = first batch row, rows, where the state
  // comes from, where it goes; a place is a row of `state` (v >= 0), nothing / zeros (-1), or
  // entry -(v + 2) of `scratch` (v <= -2)
  const int32_t* items;
  float* scratch;           // [entries, H, D, E]
  int H, D, E;
  float k_scale;
  int act;                  // 1: silu on q, k and v
  // selective variants (all optional): a decay per token and head instead of the head's constant,
  // a factor per token and head on v as it enters the state, a term skip_h * v_t added to the
  // output, and q / k shared by `kq_share` neighbouring heads (a group's q and k lie once in the
  // projection)
  const float* tok_decay;   // [T, H] or null
  const float* tok_scale;   // [T, H] or null
  const float* skip;        // [H] or null
  int kq_share;             // heads that share one q and k (1: every head its own)
  float* chunk_decay;       // [entries, H]: product of a chunk's decays, written by the pass without outputs
};

// silu with the fast exponential and division (errors of a few units in the last place of float32)
__device__ __forceinline__ float act_of(float x, int act) { return act ? __fdividef(x, 1.0f + __expf(-x)) : x; }

// DPT: state elements a thread holds (its share of D); PARTS threads share one value column;
// WARPS warps a block, which stage q and k of TB tokens at a time for all of them
template <typename T, int DPT, int PARTS, int WARPS, int TB>
__global__ void __launch_bounds__(32 * WARPS) linear_attention_kernel(LinAttnParams p) {
  constexpr int NT = 32 * WARPS;
  constexpr int COLS = NT / PARTS;             // value columns a block covers
  constexpr int DMAX = DPT * PARTS;
  // a part's DPT elements are followed by four floats of padding: the PARTS lanes of a column read
  // their own parts at once, 16 bytes each, and would otherwise all start in the same bank
  constexpr int PSTRIDE = PARTS > 1 ? DPT + 4 : DPT;
  constexpr int ROW = PARTS * PSTRIDE;
  __shared__ __align__(16) float qs[2][TB][ROW], ks[2][TB][ROW];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x;
  const int part = tid % PARTS, col = tid / PARTS;
  const int e = blockIdx.z * COLS + col;
  const int D = p.D, E = p.E, H = p.H;
  int n, t0, src, dst;
  if (p.items) {
    const int32_t* it = p.items + (size_t)r * 4;
    t0 = it[0]; n = it[1]; src = it[2]; dst = it[3];
  } else {
    n = p.q_len[r];
    t0 = p.q_start[r];
    src = dst = n > 0 ? p.slots[r] : -1;
  }
  if (n <= 0) return;
  const bool live = e < E;
  const int d0 = part * DPT;                   // this thread's first state row
  const size_t per_head = (size_t)D * E;
  auto place = [&](int v) -> float* {
    if (v == -1) return nullptr;
    return (v >= 0 ? p.state + (size_t)v * H * per_head : p.scratch + (size_t)(-(v + 2)) * H * per_head) + h * per_head;
  };
  const float* st_in = place(src);
  float* st = place(dst);
  float S[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = (st_in && live && d0 + i < D) ? st_in[(size_t)(d0 + i) * E + e] : 0.f;
  const float lam = p.decay ? p.decay[h] : 1.f;
  const float skip = p.skip ? p.skip[h] : 0.f;
  const T* qp = (const T*)p.q + (size_t)(h / p.kq_share) * D;
  const T* kp = (const T*)p.k + (size_t)(h / p.kq_share) * D;
  const T* vp = (const T*)p.v + (size_t)h * E;
  constexpr int PER = (DMAX + NT - 1) / NT;    // q and k elements of a token a thread fetches
  // a batch of TB tokens travels together: all its loads are in flight at once, and it waits in
  // registers while the batch before it is computed
  T qn[TB][PER], kn[TB][PER], vn[TB];
  float dn[TB], sn[TB];        // the tokens' decays and factors on v
  auto fetch = [&](int b) {
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
      const int t = b * TB + tt;
      const bool ok = t < n;
      const size_t row = (size_t)(t0 + (ok ? t : 0)) * p.ld;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int d = tid + i * NT;
        qn[tt][i] = (ok && d < D) ? qp[row + d] : from_float<T>(0.f);
        kn[tt][i] = (ok && d < D) ? kp[row + d] : from_float<T>(0.f);
      }
      vn[tt] = (ok && live) ? vp[row + e] : from_float<T>(0.f);
      const size_t th = (size_t)(t0 + (ok ? t : 0)) * H + h;
      dn[tt] = p.tok_decay ? p.tok_decay[th] : lam;
      sn[tt] = p.tok_scale ? p.tok_scale[th] : 1.f;
    }
  };
  float vcur[TB], xcur[TB], dcur[TB];
  float decay_product = 1.f;
  auto stage = [&](int buf) {
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int d = tid + i * NT;
        if (d < DMAX) {
          const int at = (d / DPT) * PSTRIDE + (d % DPT);
          qs[buf][tt][at] = act_of(to_float(qn[tt][i]), p.act);
          ks[buf][tt][at] = act_of(to_float(kn[tt][i]), p.act) * p.k_scale;
        }
      }
      xcur[tt] = act_of(to_float(vn[tt]), p.act);
      vcur[tt] = xcur[tt] * sn[tt];
      dcur[tt] = dn[tt];
    }
  };
  const int nb = (n + TB - 1) / TB;
  fetch(0);
  stage(0);
  if (nb > 1) fetch(1);
  for (int b = 0; b < nb; ++b) {
    // batch b is staged in buffer b & 1 (visible after this barrier); batch b + 1 waits in registers
    // and is staged into the other buffer, which batch b - 1's readers have left
    if (WARPS > 1) __syncthreads(); else __syncwarp();
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
      const int t = b * TB + tt;
      if (t >= n) break;
      const float* kb = ks[b & 1][tt] + part * PSTRIDE;
      const float* qb = qs[b & 1][tt] + part * PSTRIDE;
      const float v = vcur[tt];
      const float lam = dcur[tt];
      decay_product *= lam;
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;       // four chains: the sum's latency does not bind
      if (p.out) {
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kb + i);
          const float4 q4 = *reinterpret_cast<const float4*>(qb + i);
          S[i] = fmaf(lam, S[i], k4.x * v);
          o0 = fmaf(S[i], q4.x, o0);
          S[i + 1] = fmaf(lam, S[i + 1], k4.y * v);
          o1 = fmaf(S[i + 1], q4.y, o1);
          S[i + 2] = fmaf(lam, S[i + 2], k4.z * v);
          o2 = fmaf(S[i + 2], q4.z, o2);
          S[i + 3] = fmaf(lam, S[i + 3], k4.w * v);
          o3 = fmaf(S[i + 3], q4.w, o3);
        }
      } else {                                             // a chunk's own contribution only
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kb + i);
          S[i] = fmaf(lam, S[i], k4.x * v);
          S[i + 1] = fmaf(lam, S[i + 1], k4.y * v);
          S[i + 2] = fmaf(lam, S[i + 2], k4.z * v);
          S[i + 3] = fmaf(lam, S[i + 3], k4.w * v);
        }
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int m = 1; m < PARTS; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (p.out && live && part == 0) p.out[(size_t)(t0 + t) * H * E + (size_t)h * E + e] = fmaf(skip, xcur[tt], o);
    }
    if (b + 1 < nb) {
      stage((b + 1) & 1);
      if (b + 2 < nb) fetch(b + 2);
    }
  }
  if (live && st) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < D) st[(size_t)(d0 + i) * E + e] = S[i];
  }
  if (p.chunk_decay && dst <= -2 && tid == 0 && blockIdx.z == 0) p.chunk_decay[(size_t)(-(dst + 2)) * H + h] = decay_product;
}

// The states at the chunks' starts from the chunks' own contributions, in place (see the top).
struct ScanParams {
  float* state;
  float* scratch;
  const float* decay;
  const int32_t* desc;      // [m, 4]: state row, first scratch entry, chunks, rows of every chunk but the last
  int H, D, E;
  const float* chunk_decay; // [entries, H] or null: the chunks' own decay products (decays that differ by token)
};

__global__ void chunk_scan_kernel(ScanParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* d = p.desc + (size_t)blockIdx.x * 4;
  const int h = blockIdx.y;
  const size_t per_head = (size_t)p.D * p.E;
  const size_t i = (size_t)blockIdx.z * blockDim.x + threadIdx.x;
  if (i >= per_head) return;
  const float lam = p.decay ? p.decay[h] : 1.f;
  float lam_n = 1.f;
  if (!p.chunk_decay)
    for (int j = 0; j < d[3]; ++j) lam_n *= lam;
  float S = p.state[((size_t)d[0] * p.H + h) * per_head + i];
  for (int c = 0; c < d[2]; ++c) {
    float* u = p.scratch + ((size_t)(d[1] + c) * p.H + h) * per_head + i;
    const float own = c + 1 < d[2] ? *u : 0.f;
    if (p.chunk_decay && c + 1 < d[2]) lam_n = p.chunk_decay[(size_t)(d[1] + c) * p.H + h];
    *u = S;
    S = fmaf(lam_n, S, own);
  }
}

template <typename T, int DPT, int PARTS, int WARPS, int TB>
void launch_la(const LinAttnParams& p, int R, cudaStream_t stream) {
  constexpr int COLS = 32 * WARPS / PARTS;
  dim3 grid(R, p.H, (p.E + COLS - 1) / COLS);
  launch_k(linear_attention_kernel<T, DPT, PARTS, WARPS, TB>, grid, 32 * WARPS, 0, stream, p);
}

// 32 state elements a thread (16 for the narrowest keys); wider keys are shared by 2 to 16 threads
// of a warp, and from 4 on a block has four warps that stage q and k together.  Tokens are staged
// eight at a time (fewer where a token's keys are wide: the two buffers stay under 48 KB).
template <typename T>
int dispatch_la(const LinAttnParams& p, int R, cudaStream_t stream) {
  const int D = p.D;
  if (D <= 16) launch_la<T, 16, 1, 1, 8>(p, R, stream);
  else if (D <= 32) launch_la<T, 32, 1, 1, 8>(p, R, stream);
  else if (D <= 64) launch_la<T, 32, 2, 1, 8>(p, R, stream);
  else if (D <= 128) launch_la<T, 32, 4, 4, 8>(p, R, stream);
  else if (D <= 256) launch_la<T, 32, 8, 4, 4>(p, R, stream);
  else if (D <= 512) launch_la<T, 32, 16, 4, 2>(p, R, stream);
  else return (int)cudaErrorInvalidValue;
  return launch_status();
}
}  // namespace

PBE_EXPORT int pbe_linear_attention(const void* q, const void* k, const void* v, int ld, int dtype, float* out,
                                    float* state, const float* decay, const int32_t* q_start, const int32_t* q_len,
                                    const int32_t* slots, const int32_t* items, float* scratch, int R, int H, int D,
                                    int E, float k_scale, int act, const float* tok_decay, const float* tok_scale,
                                    const float* skip, int kq_share, float* chunk_decay, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (kq_share < 1 || H % kq_share != 0) return (int)cudaErrorInvalidValue;
  LinAttnParams p{q, k, v, ld, out, state, decay, q_start, q_len, slots, items, scratch, H, D, E, k_scale, act,
                  tok_decay, tok_scale, skip, kq_share, chunk_decay};
  return dtype == PBE_F32 ? dispatch_la<float>(p, R, stream) : dispatch_la<__nv_bfloat16>(p, R, stream);
}

PBE_EXPORT int pbe_linear_attention_scan(float* state, float* scratch, const float* decay, const int32_t* desc,
                                         int m, int H, int D, int E, const float* chunk_decay, cudaStream_t stream) {
  if (m <= 0) return 0;
  ScanParams p{state, scratch, decay, desc, H, D, E, chunk_decay};
  dim3 grid(m, H, (unsigned)(((size_t)D * E + 255) / 256));
  launch_k(chunk_scan_kernel, grid, 256, 0, stream, p);
  return launch_status();
}
