// A short causal convolution per channel over each request's rows, with the last taps - 1 inputs
// of a request carried from step to step in a state row, and the step sizes and decays of a
// selective state-space recurrence.
//
// short_conv: y[t, c] = act(b[c] + sum_j w[c, j] u[t - (taps - 1) + j, c]); u is a column slice
// of a wider projection; inputs before the rows this step brings come from the request's state
// row ([taps - 1, C] float32 per request slot, the newest input last), which holds zeros for a
// request's first tokens.  One thread per (row, channel); arithmetic in float32, the result
// rounded once.  short_conv_state then moves the state on: it is a launch of its own, because
// every row of the step may read the old state.
//
// step_sizes: dt = softplus(u + bias_h) (no clamp) and a = exp(-exp(A_h) dt) per token and head,
// float32, from a column slice of the projection.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
constexpr int MAX_TAPS = 16;

struct ConvParams {
  const void* in;            // element (row 0, channel 0) inside the projection
  int ld;                    // row stride of the projection, elements
  const float* weight;       // [C, taps]
  const float* weight_t;     // the same as [taps, C], or null (the eight-channel kernel reads it)
  const float* bias;         // [C] or null
  float* state;              // [slots, taps - 1, C]
  void* out;                 // [T, C]
  const int32_t* request_of_row;   // [T]
  const int32_t* q_start;    // [R]
  const int32_t* q_len;      // [R]
  const int32_t* slots;      // [R] state row of each request
  int T, R, C, taps;
  int act;                   // 1: silu
};

template <typename T>
__global__ void short_conv_kernel(ConvParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int r = p.request_of_row[t];
  T* out = (T*)p.out + (size_t)t * p.C + c;
  if (r < 0 || r >= p.R || p.q_len[r] <= 0) {      // a padding row of a captured step
    *out = from_float<T>(0.f);
    return;
  }
  const int i = t - p.q_start[r];                  // the row's place among the request's rows of this step
  const int taps = p.taps;
  const float* st = p.state + (size_t)p.slots[r] * (taps - 1) * p.C + c;
  const T* in = (const T*)p.in + c;
  float acc = p.bias ? p.bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int off = i - (taps - 1) + j;            // the input's place; negative: before this step
    const float u = off >= 0 ? to_float(in[(size_t)(t - (taps - 1) + j) * p.ld]) : st[(size_t)(taps - 1 + off) * p.C];
    acc = fmaf(p.weight[(size_t)c * taps + j], u, acc);
  }
  if (p.act) acc = acc / (1.0f + expf(-acc));
  *out = from_float<T>(acc);
}

// bfloat16, eight neighbouring channels a thread: one 16-byte load a tap, one 16-byte store
__global__ void short_conv_bf16x8_kernel(ConvParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= p.C) return;
  const int r = p.request_of_row[t];
  __nv_bfloat16* out = (__nv_bfloat16*)p.out + (size_t)t * p.C + c;
  if (r < 0 || r >= p.R || p.q_len[r] <= 0) {
    *reinterpret_cast<uint4*>(out) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const int i = t - p.q_start[r];
  const int taps = p.taps;
  const float* st = p.state + (size_t)p.slots[r] * (taps - 1) * p.C + c;
  const __nv_bfloat16* in = (const __nv_bfloat16*)p.in + c;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = p.bias ? p.bias[c + k] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int off = i - (taps - 1) + j;
    float u[8];
    if (off >= 0) {
      const uint4 raw = *reinterpret_cast<const uint4*>(in + (size_t)(t - (taps - 1) + j) * p.ld);
      const unsigned w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[k]));
        u[2 * k] = f.x;
        u[2 * k + 1] = f.y;
      }
    } else {
      const float* srow = st + (size_t)(taps - 1 + off) * p.C;
      const float4 a = *reinterpret_cast<const float4*>(srow), b = *reinterpret_cast<const float4*>(srow + 4);
      u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w; u[4] = b.x; u[5] = b.y; u[6] = b.z; u[7] = b.w;
    }
    const float* wrow = p.weight_t + (size_t)j * p.C + c;
    const float4 w0 = *reinterpret_cast<const float4*>(wrow), w1 = *reinterpret_cast<const float4*>(wrow + 4);
    const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = fmaf(wv[k], u[k], acc[k]);
  }
  unsigned packed[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float a = acc[2 * k], b = acc[2 * k + 1];
    if (p.act) {
      a = a / (1.0f + expf(-a));
      b = b / (1.0f + expf(-b));
    }
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    packed[k] = *reinterpret_cast<const unsigned*>(&v);
  }
  *reinterpret_cast<uint4*>(out) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

template <typename T>
__global__ void short_conv_state_kernel(ConvParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int n = p.q_len[r];
  if (n <= 0) return;
  const int keep = p.taps - 1;
  float* st = p.state + (size_t)p.slots[r] * keep * p.C + c;
  const T* in = (const T*)p.in + c;
  const int t0 = p.q_start[r];
  float fresh[MAX_TAPS];
#pragma unroll
  for (int i = 0; i < MAX_TAPS; ++i) {
    if (i < keep) {
      const int li = n - keep + i;                 // the input that becomes entry i
      fresh[i] = li >= 0 ? to_float(in[(size_t)(t0 + li) * p.ld]) : st[(size_t)(i + n) * p.C];
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_TAPS; ++i)
    if (i < keep) st[(size_t)i * p.C] = fresh[i];
}

struct StepSizeParams {
  const void* in;            // element (row 0, head 0) of the step-size columns inside the projection
  int ld;
  const float* bias;         // [H]
  const float* rate_log;     // [H]: the decay rate's logarithm
  float* dt;                 // [T, H]
  float* decay;              // [T, H]
  int T, H;
};

template <typename T>
__global__ void step_sizes_kernel(StepSizeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)p.T * p.H) return;
  const int t = (int)(idx / p.H), h = (int)(idx - (size_t)t * p.H);
  const float u = to_float(((const T*)p.in)[(size_t)t * p.ld + h]) + p.bias[h];
  const float dt = u > 20.f ? u : log1pf(expf(u));
  p.dt[idx] = dt;
  p.decay[idx] = expf(-expf(p.rate_log[h]) * dt);
}
}  // namespace

PBE_EXPORT int pbe_short_conv(const void* in, int ld, int dtype, const float* weight, const float* weight_t,
                              const float* bias, float* state,
                              void* out, const int32_t* request_of_row, const int32_t* q_start, const int32_t* q_len,
                              const int32_t* slots, int T, int R, int C, int taps, int act, int update_state,
                              cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) return (int)cudaErrorInvalidValue;
  ConvParams p{in, ld, weight, weight_t, bias, state, out, request_of_row, q_start, q_len, slots, T, R, C, taps, act};
  const int threads = C >= 256 ? 256 : 128;
  dim3 grid(T, (C + threads - 1) / threads);
  const bool vec8 = weight_t != nullptr && (((uintptr_t)weight_t) & 15) == 0 && dtype == PBE_BF16 && C % 8 == 0 && ld % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0 &&
                    (((uintptr_t)state) & 15) == 0;
  if (vec8) {
    const int th = C / 8 >= 128 ? 128 : 64;
    launch_k(short_conv_bf16x8_kernel, dim3(T, (C / 8 + th - 1) / th), th, 0, stream, p);
  } else if (dtype == PBE_F32) {
    launch_k(short_conv_kernel<float>, grid, threads, 0, stream, p);
  } else {
    launch_k(short_conv_kernel<__nv_bfloat16>, grid, threads, 0, stream, p);
  }
  int e = launch_status();
  if (e != 0 || !update_state || taps == 1) return e;
  dim3 grid2(R, (C + threads - 1) / threads);
  if (dtype == PBE_F32) launch_k(short_conv_state_kernel<float>, grid2, threads, 0, stream, p);
  else launch_k(short_conv_state_kernel<__nv_bfloat16>, grid2, threads, 0, stream, p);
  return launch_status();
}

PBE_EXPORT int pbe_step_sizes(const void* in, int ld, int dtype, const float* bias, const float* rate_log, float* dt,
                              float* decay, int T, int H, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  StepSizeParams p{in, ld, bias, rate_log, dt, decay, T, H};
  const int blocks = (int)(((size_t)T * H + 127) / 128);
  if (dtype == PBE_F32) launch_k(step_sizes_kernel<float>, blocks, 128, 0, stream, p);
  else launch_k(step_sizes_kernel<__nv_bfloat16>, blocks, 128, 0, stream, p);
  return launch_status();
}
