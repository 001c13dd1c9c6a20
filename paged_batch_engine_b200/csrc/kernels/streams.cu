// Residual streams and the norms around them.
//
// stream_norm: the residual is S parallel streams r_0..r_{S-1} per row (S = 1: the usual
// single stream).  One launch (a) folds the pending output y of the sublayer before into the
// streams, r'_j = sum_s M[s, j] r_s + beta_j y (M = 1, beta = 1 with one stream: the plain
// residual add), (b) collapses them, a = sum_j alpha_j r'_j, and (c) normalises a:
// LayerNorm ((a - mean) / sqrt(mean((a - mean)^2) + eps) * g + b, the variance from the
// deviations, two passes over the row in shared memory) or RMSNorm (a / sqrt(mean(a^2) + eps)
// * g).  With a row index the rows are gathered and the streams are left alone (the final
// norm on the wanted rows).  Streams, sums and statistics are float32.
//
// branch_rms_mean: the mean of up to four branches, each divided by its root mean square
// over the row and multiplied by a gain of its own.
//
// gated_rms: o / rms(o) (over the whole row or over each head's slice), times an optional
// gain, times sigmoid(g) or silu(g) of a gate that lies in a wider matrix; or, gate first, the
// gated values o * act(g) divided by their own root mean square, times the gain.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
constexpr int MAX_STREAMS = 8;

struct StreamNormParams {
  float* streams;          // [T, S, W]
  const void* y;           // [T, W] pending sublayer output, or null
  const float* mix;        // [S, S] indexed [from, to]
  const float* beta;       // [S]
  const float* alpha;      // [S]
  const float* gain;       // [W]
  const float* bias;       // [W] or null
  void* out;               // [n, W]
  const int32_t* rows;     // [n] or null
  int S, W;
  float eps;
  int rms;                 // 1: RMSNorm, 0: LayerNorm
};

template <typename TY, typename TO>
__global__ void stream_norm_kernel(StreamNormParams p) {
  __shared__ float red[33];
  __shared__ float coef[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
  extern __shared__ __align__(16) float row[];       // W floats: the collapsed row
  pdl_launch_dependents();
  const int S = p.S, W = p.W;
  float* mix = coef;
  float* beta = coef + MAX_STREAMS * MAX_STREAMS;
  float* alpha = beta + MAX_STREAMS;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix[i] = p.mix[i];
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    beta[i] = p.beta[i];
    alpha[i] = p.alpha[i];
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const int src = p.rows ? p.rows[r] : r;
  float* res = p.streams + (size_t)src * S * W;
  const TY* y = p.y ? (const TY*)p.y + (size_t)src * W : nullptr;
  const bool write_back = p.rows == nullptr && y != nullptr;
  float sum = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float x[MAX_STREAMS], z[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) x[s] = s < S ? res[(size_t)s * W + c] : 0.f;
    float a = 0.f;
    if (y) {
      const float yc = to_float(y[c]);
#pragma unroll
      for (int j = 0; j < MAX_STREAMS; ++j) {
        if (j < S) {
          float v = 0.f;
          for (int s = 0; s < S; ++s) v = fmaf(mix[s * S + j], x[s], v);
          z[j] = fmaf(beta[j], yc, v);
          if (write_back) res[(size_t)j * W + c] = z[j];
        }
      }
#pragma unroll
      for (int j = 0; j < MAX_STREAMS; ++j)
        if (j < S) a = fmaf(alpha[j], z[j], a);
    } else {
#pragma unroll
      for (int j = 0; j < MAX_STREAMS; ++j)
        if (j < S) a = fmaf(alpha[j], x[j], a);
    }
    row[c] = a;
    sum += p.rms ? a * a : a;
  }
  const float total = block_sum(sum, red);
  TO* o = (TO*)p.out + (size_t)r * W;
  if (p.rms) {
    const float scale = rsqrtf(total / (float)W + p.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) o[c] = from_float<TO>((p.gain[c] * row[c]) * scale);
    return;
  }
  const float mean = total / (float)W;
  float sq = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float d = row[c] - mean;
    sq += d * d;
  }
  const float var = block_sum(sq, red) / (float)W;
  const float scale = 1.0f / sqrtf(var + p.eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = (row[c] - mean) * scale * p.gain[c];
    if (p.bias) v += p.bias[c];
    o[c] = from_float<TO>(v);
  }
}

struct BranchParams {
  const void* x[4];        // each [T, W]
  const float* gain[4];    // each [W]
  void* out;               // [T, W]
  int n, W;
  float eps;
};

template <typename T>
__global__ void branch_rms_mean_kernel(BranchParams p) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, W = p.W;
  float scale[4];
  for (int b = 0; b < p.n; ++b) {
    const T* x = (const T*)p.x[b] + (size_t)t * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = to_float(x[c]);
      ss += v * v;
    }
    scale[b] = rsqrtf(block_sum(ss, red) / (float)W + p.eps);
  }
  const float inv_n = 1.0f / (float)p.n;
  T* o = (T*)p.out + (size_t)t * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float a = 0.f;
    for (int b = 0; b < p.n; ++b)
      a += to_float(((const T*)p.x[b])[(size_t)t * W + c]) * scale[b] * p.gain[b][c];
    o[c] = from_float<T>(a * inv_n);
  }
}

struct GatedRmsParams {
  const float* o;          // [T, H * E]
  const void* gate;        // first gate element of row 0; row stride ld_gate elements
  const float* gain;       // [H * E] or null
  void* out;               // [T, H * E]
  int ld_gate, H, E;
  float eps;
  int per_head;            // 1: each head's E values have a root mean square of their own
  int gate_act;            // 0: sigmoid, 1: silu
  int gate_first;          // 1: the gate multiplies o before the root mean square is taken (of the gated values)
};

template <typename T>
__global__ void gated_rms_kernel(GatedRmsParams p) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, H = p.H, E = p.E, N = H * E;
  const float* o = p.o + (size_t)t * N;
  const T* g = (const T*)p.gate + (size_t)t * p.ld_gate;
  T* out = (T*)p.out + (size_t)t * N;
  auto gate_of = [&](int c) {
    const float gv = to_float(g[c]);
    const float sg = 1.0f / (1.0f + expf(-gv));
    return p.gate_act ? gv * sg : sg;
  };
  // what the root mean square is taken of: o itself, or (gate_first) o times its gate
  auto value = [&](int c) { return p.gate_first ? o[c] * gate_of(c) : o[c]; };
  auto finish = [&](int c, float scale) {
    float v = value(c) * scale;
    if (p.gain) v *= p.gain[c];
    out[c] = from_float<T>(p.gate_first ? v : v * gate_of(c));
  };
  if (p.per_head) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int h = warp; h < H; h += nw) {
      float ss = 0.f;
      for (int e = lane; e < E; e += 32) {
        const float v = value(h * E + e);
        ss += v * v;
      }
      const float scale = rsqrtf(warp_sum(ss) / (float)E + p.eps);
      for (int e = lane; e < E; e += 32) finish(h * E + e, scale);
    }
    return;
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    const float v = value(c);
    ss += v * v;
  }
  const float scale = rsqrtf(block_sum(ss, red) / (float)N + p.eps);
  for (int c = threadIdx.x; c < N; c += blockDim.x) finish(c, scale);
}
}  // namespace

PBE_EXPORT int pbe_stream_norm(float* streams, const void* y, int y_dtype, const float* mix, const float* beta,
                               const float* alpha, const float* gain, const float* bias, void* out, int out_dtype,
                               const int32_t* rows, int n, int S, int W, float eps, int rms, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (S < 1 || S > MAX_STREAMS) return (int)cudaErrorInvalidValue;
  StreamNormParams p{streams, y, mix, beta, alpha, gain, bias, out, rows, S, W, eps, rms};
  const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  const size_t smem = sizeof(float) * (size_t)W;
  cudaError_t e;
#define PBE_SN(TY, TO)                                                                                  \
  do {                                                                                                  \
    static int opted = 0;                                                                               \
    if (smem > 48 * 1024 && opted < (int)smem) {                                                        \
      cudaFuncSetAttribute(stream_norm_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      opted = (int)smem;                                                                                \
    }                                                                                                   \
    e = launch_k(stream_norm_kernel<TY, TO>, n, threads, smem, stream, p);                              \
  } while (0)
  const bool yb = y != nullptr && y_dtype == PBE_BF16;
  if (out_dtype == PBE_F32) {
    if (yb) PBE_SN(__nv_bfloat16, float); else PBE_SN(float, float);
  } else {
    if (yb) PBE_SN(__nv_bfloat16, __nv_bfloat16); else PBE_SN(float, __nv_bfloat16);
  }
#undef PBE_SN
  (void)e;
  return launch_status();
}

PBE_EXPORT int pbe_branch_rms_mean(const void* const* x, const float* const* gain, int n, void* out, int dtype,
                                   int T, int W, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n < 1 || n > 4) return (int)cudaErrorInvalidValue;
  BranchParams p{};
  for (int b = 0; b < n; ++b) {
    p.x[b] = x[b];
    p.gain[b] = gain[b];
  }
  p.out = out; p.n = n; p.W = W; p.eps = eps;
  const int threads = W >= 512 ? 256 : 128;
  if (dtype == PBE_F32) launch_k(branch_rms_mean_kernel<float>, T, threads, 0, stream, p);
  else launch_k(branch_rms_mean_kernel<__nv_bfloat16>, T, threads, 0, stream, p);
  return launch_status();
}

PBE_EXPORT int pbe_gated_rms(const float* o, const void* gate, int ld_gate, const float* gain, void* out, int dtype,
                             int T, int H, int E, float eps, int per_head, int gate_act, int gate_first,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  GatedRmsParams p{o, gate, gain, out, ld_gate, H, E, eps, per_head, gate_act, gate_first};
  const int threads = H * E >= 512 ? 256 : 128;
  if (dtype == PBE_F32) launch_k(gated_rms_kernel<float>, T, threads, 0, stream, p);
  else launch_k(gated_rms_kernel<__nv_bfloat16>, T, threads, 0, stream, p);
  return launch_status();
}
