// Softmax attention over a sliding window of tokens plus mean-pooled blocks of the tokens
// before it, with the heads' probabilities mixed by a matrix ("talking heads" after the
// softmax).  Three kernels:
//
// qk_prepare: per token, an optional RMS norm over the WHOLE query projection and over the
//   whole key projection (all heads at once, one gain per element), rotary position encoding
//   on the first `rot` dimensions of every head (neighbouring pairs (2i, 2i+1), or none), the
//   query out, key and value into the token pages.
// pool_blocks: a token at position p with (p + 1) % pool == 0 completes block p / pool; its
//   pooled key and value are the means of the block's keys and values as the token pages hold
//   them, written to the entry of the block in the pooled pages (one entry per `pool` tokens).
// pooled_attention: a row at position p sees the pooled blocks b with b*pool + pool - 1 <=
//   p - window and the tokens p - window + 1 .. p, in one softmax.  A block of threads takes
//   BM consecutive rows of a request and all heads.  Pass 1 walks the key tiles and keeps each
//   (row, head)'s running maximum and sum; pass 2 walks them again, turns the scores into
//   normalised probabilities, mixes them across heads, w'_h = sum_g M[h, g] w_g, and adds
//   w'_h times the values of head h's key/value head.  The normalised probabilities of all
//   heads are needed before any value is weighted, hence the two passes; the scores are
//   computed by the same arithmetic in both, so the maximum of pass 1 is exact in pass 2.
//   All arithmetic is float32.
//
// Compile with -DPBE_PA_F32=1 for float32 tensors, 0 for bfloat16: a library holds one of them.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

#ifndef PBE_PA_F32
#error "PBE_PA_F32 must be defined (1: float32, 0: bfloat16)"
#endif

namespace {
#if PBE_PA_F32
using PaT = float;
constexpr int PA_DTYPE = PBE_F32;
#else
using PaT = __nv_bfloat16;
constexpr int PA_DTYPE = PBE_BF16;
#endif
// ------------------------------------------------------------------ qk_prepare
struct QkPrepParams {
  const void* q;            // row 0 of each inside the projection, row stride ld elements
  const void* k;
  const void* v;
  int ld;
  const float* q_gain;      // [H * D] or null: no norm
  const float* k_gain;      // [G * D] or null
  const float* inv_freq;    // [rot / 2] or null
  const int32_t* positions; // [T]
  const int32_t* slots;     // [T] page * page_tokens + offset in the token pages
  void* q_out;              // [T, H * D]
  void* k_pages;            // [page][G][page_tokens][D] or null: nothing is written
  void* v_pages;            // [page][G][page_tokens][E]
  int H, G, D, E, rot, page_tokens;
  float eps;
};

template <typename T>
__global__ void qk_prepare_kernel(QkPrepParams p) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int H = p.H, G = p.G, D = p.D, E = p.E, PT = p.page_tokens;
  const T* q = (const T*)p.q + (size_t)t * p.ld;
  const T* k = (const T*)p.k + (size_t)t * p.ld;
  const T* v = (const T*)p.v + (size_t)t * p.ld;
  float q_scale = 1.f, k_scale = 1.f;
  if (p.q_gain) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
      const float x = to_float(q[i]);
      ss += x * x;
    }
    q_scale = rsqrtf(block_sum(ss, red) / (float)(H * D) + p.eps);
  }
  if (p.k_gain) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
      const float x = to_float(k[i]);
      ss += x * x;
    }
    k_scale = rsqrtf(block_sum(ss, red) / (float)(G * D) + p.eps);
  }
  const float pos = (float)p.positions[t];
  // a negative slot (the padding rows of a captured step): nothing is written
  const int slot = p.slots ? p.slots[t] : -1;
  const bool store = slot >= 0;
  const int page = store ? slot / PT : 0, off = store ? slot - page * PT : 0;
  const int half = D / 2;       // pairs per head (D is even)
  T* qo = (T*)p.q_out + (size_t)t * H * D;
  // pairs of the query heads, then of the key heads
  for (int i = threadIdx.x; i < (H + G) * half; i += blockDim.x) {
    const bool is_q = i < H * half;
    const int j = is_q ? i : i - H * half;
    const int head = j / half, pr = j - head * half;
    const int e0 = head * D + 2 * pr;
    const T* src = is_q ? q : k;
    const float* gain = is_q ? p.q_gain : p.k_gain;
    const float sc = is_q ? q_scale : k_scale;
    float a = to_float(src[e0]), b = to_float(src[e0 + 1]);
    if (gain) {
      a = a * sc * gain[e0];
      b = b * sc * gain[e0 + 1];
    }
    if (p.inv_freq && 2 * pr < p.rot) {
      float sn, cs;
      sincosf(pos * p.inv_freq[pr], &sn, &cs);
      const float ra = a * cs - b * sn, rb = b * cs + a * sn;
      a = ra;
      b = rb;
    }
    if (is_q) {
      qo[e0] = from_float<T>(a);
      qo[e0 + 1] = from_float<T>(b);
    } else if (p.k_pages && store) {
      T* dst = (T*)p.k_pages + (((size_t)page * G + head) * PT + off) * D + 2 * pr;
      dst[0] = from_float<T>(a);
      dst[1] = from_float<T>(b);
    }
  }
  if (p.v_pages && store) {
    for (int i = threadIdx.x; i < G * E; i += blockDim.x) {
      const int head = i / E, e = i - head * E;
      ((T*)p.v_pages)[(((size_t)page * G + head) * PT + off) * E + e] = v[i];
    }
  }
}

// ------------------------------------------------------------------ pool_blocks
struct PoolParams {
  const void* k_tok;        // [page][G][page_tokens][D]
  const void* v_tok;        // [page][G][page_tokens][E]
  void* k_pool;             // the same layouts, one entry per block
  void* v_pool;
  const int32_t* positions; // [T]
  const int32_t* request;   // [T] row of the block tables
  const int32_t* bt_tok;
  const int32_t* bt_pool;
  int bt_tok_stride, bt_pool_stride;
  int G, D, E, page_tokens, pool;
};

template <typename T>
__global__ void pool_blocks_kernel(PoolParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  const int pos = p.positions[t];
  if ((pos + 1) % p.pool != 0) return;
  const int PT = p.page_tokens, G = p.G, D = p.D, E = p.E;
  const int r = p.request[t];
  const int block = pos / p.pool;
  const int32_t* bt = p.bt_tok + (size_t)r * p.bt_tok_stride;
  const int ppage = p.bt_pool[(size_t)r * p.bt_pool_stride + block / PT];
  const int poff = block % PT;
  if (ppage < 0) return;
  const float inv = 1.0f / (float)p.pool;
  for (int c = threadIdx.x; c < D + E; c += blockDim.x) {
    const bool is_k = c < D;
    const int w = is_k ? D : E, col = is_k ? c : c - D;
    const T* src = (const T*)(is_k ? p.k_tok : p.v_tok);
    float sum = 0.f;
    for (int j = 0; j < p.pool; ++j) {
      const int tok = block * p.pool + j;
      const int page = bt[tok / PT];
      if (page >= 0) sum += to_float(src[(((size_t)page * G + g) * PT + tok % PT) * w + col]);
    }
    T* dst = (T*)(is_k ? p.k_pool : p.v_pool);
    dst[(((size_t)ppage * G + g) * PT + poff) * w + col] = from_float<T>(sum * inv);
  }
}

// ------------------------------------------------------------------ pooled_attention
struct PoolAttnParams {
  const void* q;            // [T, H * D]
  const void* k_tok;
  const void* v_tok;
  const void* k_pool;
  const void* v_pool;
  void* out;                // [T, H * E]
  const float* talk;        // [H, H] (row h: the weights of head h's mixture) or null
  const int32_t* tiles;     // [n, 3]: request, first batch row, rows
  const int32_t* q_start;   // [R]
  const int32_t* q_len;
  const int32_t* seq_len;
  const int32_t* bt_tok;
  const int32_t* bt_pool;
  int bt_tok_stride, bt_pool_stride;
  int H, G, D, E, page_tokens, window, pool, BN;
  float scale;
  // the keys of a row tile cut into splits of `split_tiles` key tiles, a block each (grid.y):
  int split_tiles, splits;
  float* part_ml;           // [tiles][splits][BM * H][2]: maximum and sum of each split
  float* stats;             // [tiles][BM * H][2]: the same over all splits
  float* part_o;            // [tiles][splits][BM * H * E]: a split's share of the output
  int mode;                 // 0, 1 or 2: see the kernel
};

constexpr int PA_THREADS = 512;   // sixteen warps: one block a multiprocessor has to hide its own latencies (256: 6.6 ms, 512: 4.3 ms for a 2,048-token prompt)
constexpr int PA_ACC = 32;      // outputs a thread accumulates at most

__device__ __forceinline__ void unpack16(const uint4& r, float* f, float) {
  f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
}
__device__ __forceinline__ void unpack16(const uint4& r, float* f, __nv_bfloat16) {
  const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// A tile of BN keys (or values), all G key/value heads of each, from the pages into shared memory
// as float32 rows of `stride` floats: row j = [head 0's `width` elements, head 1's, ...]; keys that
// do not exist (base < 0) become zeros.  Rows whose width fills 16-byte pieces travel as such,
// four pieces a thread in flight.
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int stride, const T* src, const long long* base, int BN, int G,
                                          int width, int PT) {
  constexpr int VEC = 16 / (int)sizeof(T);
  if (width % VEC == 0) {
    const int wv = width / VEC, per_key = G * wv, total = BN * per_key;
    constexpr int U = 4;
    for (int i0 = threadIdx.x; i0 < total; i0 += PA_THREADS * U) {
      uint4 r[U];
      int at[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * PA_THREADS;
        at[u] = -1;
        r[u] = make_uint4(0u, 0u, 0u, 0u);
        if (i < total) {
          const int j = i / per_key, c = i - j * per_key;
          const int g = c / wv, dv = c - g * wv;
          at[u] = j * stride + g * width + dv * VEC;
          const long long b = base[j];
          if (b >= 0) r[u] = *reinterpret_cast<const uint4*>(src + (b + (long long)g * PT) * width + dv * VEC);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (at[u] >= 0) {
          float f[VEC];
          unpack16(r[u], f, T());
#pragma unroll
          for (int x = 0; x < VEC; ++x) dst[at[u] + x] = f[x];
        }
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < BN * G * width; i += PA_THREADS) {
    const int j = i / (G * width), c = i - j * (G * width);
    const int g = c / width, d = c - g * width;
    const long long b = base[j];
    dst[j * stride + c] = b >= 0 ? to_float(src[(b + (long long)g * PT) * width + d]) : 0.f;
  }
}

// MODE 0: a block walks all key tiles of its row tile twice (statistics, then values).
// MODE 1: a block walks its split of the key tiles once and leaves the split's statistics.
// MODE 2: a block takes the statistics over all splits (made by pa_combine_kernel), walks its
//         split and leaves its share of the output; the shares are plain addends, since every
//         probability is already normalised (pa_sum_kernel adds them).
template <typename T, int BM>
__global__ void __launch_bounds__(PA_THREADS) pooled_attention_kernel(PoolAttnParams p) {
  const int MODE = p.mode;
  extern __shared__ __align__(16) float smem[];
  const int H = p.H, G = p.G, D = p.D, E = p.E, PT = p.page_tokens, BN = p.BN;
  const int rep = H / G;
  const int KS = G * D + 1;                  // padded key row
  float* Qs = smem;                          // [BM][H * D], scaled
  float* Ks = Qs + ((BM * H * D + 3) & ~3);  // [BN][KS]; what follows stays on 16-byte boundaries
  float* Vs = Ks + BN * KS;                  // [BN][G * E]
  float* Ss = Vs + BN * G * E;               // [BM][H][BN] scores, then probabilities
  float* Ws = Ss + BM * H * BN;              // [BM][H][BN] mixed probabilities
  float* Ms = Ws + BM * H * BN;              // [BM][H] running maximum
  float* Ls = Ms + BM * H;                   // [BM][H] running sum
  float* Tk = Ls + BM * H;                   // [H][H]
  // [BN]: (page * G * page_tokens + offset) of key j, -1: no such key; on an 8-byte boundary
  long long* base = reinterpret_cast<long long*>(smem + (((Tk - smem) + H * H + 1) & ~(ptrdiff_t)1));
  pdl_launch_dependents();
  if (p.talk)
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) Tk[i] = p.talk[i];
  pdl_wait();
  const int32_t* tile = p.tiles + (size_t)blockIdx.x * 3;
  const int r = tile[0], row0 = tile[1], rows = tile[2];
  const int pos0 = p.seq_len[r] - p.q_len[r] + (row0 - p.q_start[r]);     // position of the tile's first row
  const int pos_last = pos0 + rows - 1;
  const int W = p.window, PL = p.pool;
  // pooled blocks the last row sees, tokens from the first row's window on
  const int nb_max = (PL > 0 && pos_last - W + 1 > 0) ? (pos_last - W + 1) / PL : 0;
  const int tok_lo = max(0, pos0 - W + 1);
  const int n_tok = pos_last - tok_lo + 1;
  const int pool_tiles = (nb_max + BN - 1) / BN, tok_tiles = (n_tok + BN - 1) / BN;
  const int32_t* bt_tok = p.bt_tok + (size_t)r * p.bt_tok_stride;
  const int32_t* bt_pool = p.bt_pool ? p.bt_pool + (size_t)r * p.bt_pool_stride : nullptr;

  if (MODE != 0 && (int)blockIdx.y * p.split_tiles >= pool_tiles + tok_tiles) {
    // a split beyond this row tile's keys: neutral statistics, a share of zeros
    if (MODE == 1) {
      float* ml = p.part_ml + (((size_t)blockIdx.x * p.splits + blockIdx.y) * BM * H) * 2;
      for (int i = threadIdx.x; i < BM * H; i += blockDim.x) {
        ml[2 * i] = -INFINITY;
        ml[2 * i + 1] = 0.f;
      }
    } else {
      float* po = p.part_o + ((size_t)blockIdx.x * p.splits + blockIdx.y) * BM * H * E;
      for (int i = threadIdx.x; i < BM * H * E; i += blockDim.x) po[i] = 0.f;
    }
    return;
  }
  for (int i = threadIdx.x; i < BM * H * D; i += blockDim.x) {
    const int row = i / (H * D), c = i - row * (H * D);
    Qs[i] = row < rows ? to_float(((const T*)p.q)[(size_t)(row0 + row) * H * D + c]) * p.scale : 0.f;
  }
  for (int i = threadIdx.x; i < BM * H; i += blockDim.x) {
    if (MODE == 2) {
      const float* st = p.stats + ((size_t)blockIdx.x * BM * H + i) * 2;
      Ms[i] = st[0];
      Ls[i] = st[1];
    } else {
      Ms[i] = -INFINITY;
      Ls[i] = 0.f;
    }
  }
  float acc[PA_ACC];
#pragma unroll
  for (int i = 0; i < PA_ACC; ++i) acc[i] = 0.f;
  const int n_out = BM * H * E;
  const int all_tiles = pool_tiles + tok_tiles;
  const int kt_lo = MODE == 0 ? 0 : min(all_tiles, (int)blockIdx.y * p.split_tiles);
  const int kt_hi = MODE == 0 ? all_tiles : min(all_tiles, kt_lo + p.split_tiles);

  for (int pass = (MODE == 2 ? 1 : 0); pass < (MODE == 1 ? 1 : 2); ++pass) {
    for (int kt = kt_lo; kt < kt_hi; ++kt) {
      const bool pooled = kt < pool_tiles;
      const int first = pooled ? kt * BN : tok_lo + (kt - pool_tiles) * BN;    // block or token index of key 0
      const int limit = pooled ? nb_max : pos_last + 1;
      __syncthreads();      // the tile before is consumed (and Qs, Ms, Ls are written, first time)
      if (threadIdx.x < BN) {
        const int idx = first + threadIdx.x;
        long long b = -1;
        if (idx < limit) {
          const int page = pooled ? bt_pool[idx / PT] : bt_tok[idx / PT];
          if (page >= 0) b = ((long long)page * G * PT + idx % PT);
        }
        base[threadIdx.x] = b;
      }
      __syncthreads();
      const T* kc = (const T*)(pooled ? p.k_pool : p.k_tok);
      load_tile<T>(Ks, KS, kc, base, BN, G, D, PT);
      if (pass == 1) load_tile<T>(Vs, G * E, (const T*)(pooled ? p.v_pool : p.v_tok), base, BN, G, E, PT);
      __syncthreads();
      // scores of every (row, head) against the tile's keys; -inf where the row does not see the key
      for (int i = threadIdx.x; i < BM * H * BN; i += blockDim.x) {
        const int j = i % BN, rh = i / BN;
        const int h = rh % H, row = rh / H;
        const int pos = pos0 + row;
        const int idx = first + j;
        bool vis = row < rows && base[j] >= 0;
        if (pooled) vis = vis && (idx * PL + PL - 1 <= pos - W);
        else vis = vis && idx <= pos && idx > pos - W;
        float s = -INFINITY;
        if (vis) {
          const float* qr = Qs + (size_t)row * H * D + h * D;
          const float* kr = Ks + j * KS + (h / rep) * D;
          float a = 0.f;
          if ((D & 3) == 0) {
            for (int d = 0; d < D; d += 4) {
              const float4 q4 = *reinterpret_cast<const float4*>(qr + d);
              a = fmaf(q4.x, kr[d], a);
              a = fmaf(q4.y, kr[d + 1], a);
              a = fmaf(q4.z, kr[d + 2], a);
              a = fmaf(q4.w, kr[d + 3], a);
            }
          } else {
            for (int d = 0; d < D; ++d) a = fmaf(qr[d], kr[d], a);
          }
          s = a;
        }
        Ss[i] = s;
      }
      __syncthreads();
      if (pass == 0) {
        // a warp per (row, head), a key per lane (BN <= 32)
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int rh = warp; rh < BM * H; rh += PA_THREADS / 32) {
          const float sc = lane < BN ? Ss[(size_t)rh * BN + lane] : -INFINITY;
          const float m = Ms[rh];
          const float mx = fmaxf(m, warp_max(sc));
          if (mx == -INFINITY) continue;          // the same for the whole warp
          const float sum = warp_sum(expf(sc - mx));
          if (lane == 0) {
            Ls[rh] = Ls[rh] * expf(m - mx) + sum;
            Ms[rh] = mx;
          }
        }
        continue;
      }
      for (int i = threadIdx.x; i < BM * H * BN; i += blockDim.x) {
        const int rh = i / BN;
        const float s = Ss[i];
        Ss[i] = s == -INFINITY ? 0.f : expf(s - Ms[rh]) / Ls[rh];
      }
      __syncthreads();
      const float* Wp = Ss;
      if (p.talk) {
        for (int i = threadIdx.x; i < BM * H * BN; i += blockDim.x) {
          const int j = i % BN, rh = i / BN;
          const int h = rh % H, row = rh / H;
          const float* pr = Ss + (size_t)row * H * BN + j;
          float a = 0.f;
          for (int g = 0; g < H; ++g) a = fmaf(Tk[h * H + g], pr[g * BN], a);
          Ws[i] = a;
        }
        Wp = Ws;
        __syncthreads();
      }
#pragma unroll
      for (int u = 0; u < PA_ACC; ++u) {
        const int o = threadIdx.x + u * PA_THREADS;
        if (o < n_out) {
          const int e = o % E, rh = o / E;
          const int h = rh % H;
          const float* w = Wp + (size_t)rh * BN;
          const float* vcol = Vs + (h / rep) * E + e;
          float a = acc[u];
          const int vs = G * E;
          for (int j = 0; j < BN; j += 4) {          // BN is a multiple of 4
            const float4 w4 = *reinterpret_cast<const float4*>(w + j);
            a = fmaf(w4.x, vcol[j * vs], a);
            a = fmaf(w4.y, vcol[(j + 1) * vs], a);
            a = fmaf(w4.z, vcol[(j + 2) * vs], a);
            a = fmaf(w4.w, vcol[(j + 3) * vs], a);
          }
          acc[u] = a;
        }
      }
    }
  }
  if (MODE == 1) {
    __syncthreads();
    float* ml = p.part_ml + (((size_t)blockIdx.x * p.splits + blockIdx.y) * BM * H) * 2;
    for (int i = threadIdx.x; i < BM * H; i += blockDim.x) {
      ml[2 * i] = Ms[i];
      ml[2 * i + 1] = Ls[i];
    }
  } else if (MODE == 2) {
    float* po = p.part_o + ((size_t)blockIdx.x * p.splits + blockIdx.y) * n_out;
#pragma unroll
    for (int u = 0; u < PA_ACC; ++u) {
      const int o = threadIdx.x + u * PA_THREADS;
      if (o < n_out) po[o] = acc[u];
    }
  } else {
#pragma unroll
    for (int u = 0; u < PA_ACC; ++u) {
      const int o = threadIdx.x + u * PA_THREADS;
      if (o < n_out) {
        const int c = o % (H * E), row = o / (H * E);
        if (row < rows) ((T*)p.out)[(size_t)(row0 + row) * H * E + c] = from_float<T>(acc[u]);
      }
    }
  }
}

// The statistics of a row tile over all its splits: m = max m_s, l = sum l_s e^(m_s - m).
__global__ void pa_combine_kernel(const float* part_ml, float* stats, int splits, int per_tile) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= per_tile) return;
  const float* ml = part_ml + ((size_t)blockIdx.x * splits * per_tile + i) * 2;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[(size_t)s * per_tile * 2]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = ml[(size_t)s * per_tile * 2];
    if (ms != -INFINITY) l += ml[(size_t)s * per_tile * 2 + 1] * expf(ms - m);
  }
  float* st = stats + ((size_t)blockIdx.x * per_tile + i) * 2;
  st[0] = m;
  st[1] = l;
}

// out = sum over the splits of their shares, in split order.
template <typename T>
__global__ void pa_sum_kernel(const float* part_o, void* out, const int32_t* tiles, int splits, int n_out, int HE) {
  pdl_launch_dependents();
  pdl_wait();
  const int o = blockIdx.y * blockDim.x + threadIdx.x;
  if (o >= n_out) return;
  const int32_t* tile = tiles + (size_t)blockIdx.x * 3;
  const int row = o / HE, c = o - row * HE;
  if (row >= tile[2]) return;
  const float* po = part_o + (size_t)blockIdx.x * splits * n_out + o;
  float a = 0.f;
  for (int s = 0; s < splits; ++s) a += po[(size_t)s * n_out];
  ((T*)out)[(size_t)(tile[1] + row) * HE + c] = from_float<T>(a);
}

template <typename T, int BM>
int launch_pa(PoolAttnParams p, int mode, int n_tiles, size_t smem, cudaStream_t stream) {
  static size_t opted = 0;
  if (smem > 48 * 1024 && opted < smem) {
    cudaFuncSetAttribute(pooled_attention_kernel<T, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    opted = smem;
  }
  p.mode = mode;
  dim3 grid(n_tiles, mode == 0 ? 1 : p.splits);
  launch_k(pooled_attention_kernel<T, BM>, grid, PA_THREADS, smem, stream, p);
  return launch_status();
}

template <typename T, int BM>
int run_pa(const PoolAttnParams& p, int n_tiles, size_t smem, cudaStream_t stream) {
  if (p.splits <= 1) return launch_pa<T, BM>(p, 0, n_tiles, smem, stream);
  int rc = launch_pa<T, BM>(p, 1, n_tiles, smem, stream);
  if (rc) return rc;
  const int per_tile = BM * p.H;
  launch_k(pa_combine_kernel, dim3(n_tiles, (per_tile + 127) / 128), 128, 0, stream, (const float*)p.part_ml, p.stats,
           p.splits, per_tile);
  if ((rc = launch_status())) return rc;
  if ((rc = launch_pa<T, BM>(p, 2, n_tiles, smem, stream))) return rc;
  const int n_out = BM * p.H * p.E;
  launch_k(pa_sum_kernel<T>, dim3(n_tiles, (n_out + 255) / 256), 256, 0, stream, (const float*)p.part_o, p.out, p.tiles,
           p.splits, n_out, p.H * p.E);
  return launch_status();
}

size_t pa_smem(int BM, int BN, int H, int G, int D, int E) {
  size_t f = (((size_t)BM * H * D + 3) & ~(size_t)3) + (size_t)BN * (G * D + 1) + (size_t)BN * G * E +
             2 * (size_t)BM * H * BN +
             2 * (size_t)BM * H + (size_t)H * H;
  f = (f + 1) & ~(size_t)1;
  return f * sizeof(float) + (size_t)BN * sizeof(long long);
}
}  // namespace

PBE_EXPORT int pbe_qk_prepare(const void* q, const void* k, const void* v, int ld, const float* q_gain,
                              const float* k_gain, const float* inv_freq, const int32_t* positions,
                              const int32_t* slots, void* q_out, void* k_pages, void* v_pages, int T, int H, int G,
                              int D, int E, int rot, int page_tokens, float eps, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 2) return (int)cudaErrorInvalidValue;
  QkPrepParams p{q, k, v, ld, q_gain, k_gain, inv_freq, positions, slots, q_out, k_pages, v_pages,
                 H, G, D, E, rot, page_tokens, eps};
  const int threads = (H + G) * D >= 2048 ? 256 : 128;
  if (dtype != PA_DTYPE) return (int)cudaErrorInvalidValue;
  launch_k(qk_prepare_kernel<PaT>, T, threads, 0, stream, p);
  return launch_status();
}

PBE_EXPORT int pbe_pool_blocks(const void* k_tok, const void* v_tok, void* k_pool, void* v_pool,
                               const int32_t* positions, const int32_t* request, const int32_t* bt_tok,
                               int bt_tok_stride, const int32_t* bt_pool, int bt_pool_stride, int T, int G, int D,
                               int E, int page_tokens, int pool, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  PoolParams p{k_tok, v_tok, k_pool, v_pool, positions, request, bt_tok, bt_pool, bt_tok_stride, bt_pool_stride,
               G, D, E, page_tokens, pool};
  dim3 grid(T, G);
  const int threads = D + E >= 256 ? 256 : (D + E >= 128 ? 128 : 64);
  if (dtype != PA_DTYPE) return (int)cudaErrorInvalidValue;
  launch_k(pool_blocks_kernel<PaT>, grid, threads, 0, stream, p);
  return launch_status();
}

// Keys per key tile for a row tile of that many rows (what the launcher will choose).
PBE_EXPORT int pbe_pooled_attention_key_tile(int tile_rows, int H, int G, int D, int E) {
  int BN = 32;
  while (BN > 4 && pa_smem(tile_rows, BN, H, G, D, E) > 200 * 1024) BN >>= 1;
  return BN;
}

// The largest row tile (1, 4 or 16) whose outputs fit a block's accumulators.
PBE_EXPORT int pbe_pooled_attention_tile_rows(int H, int E, int want) {
  int bm = 16;
  while (bm > 1 && (bm > want || (long long)bm * H * E > (long long)PA_ACC * PA_THREADS)) bm >>= 2;
  return (long long)bm * H * E > (long long)PA_ACC * PA_THREADS ? 0 : bm;
}

PBE_EXPORT int pbe_pooled_attention(const void* q, const void* k_tok, const void* v_tok, const void* k_pool,
                                    const void* v_pool, void* out, const float* talk, const int32_t* tiles,
                                    int n_tiles, int tile_rows, const int32_t* q_start, const int32_t* q_len,
                                    const int32_t* seq_len, const int32_t* bt_tok, int bt_tok_stride,
                                    const int32_t* bt_pool, int bt_pool_stride, int H, int G, int D, int E,
                                    int page_tokens, int window, int pool, float scale, int dtype, int splits,
                                    int split_tiles, float* part_ml, float* stats, float* part_o,
                                    cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (H % G || (long long)tile_rows * H * E > (long long)PA_ACC * PA_THREADS) return (int)cudaErrorInvalidValue;
  int BN = 32;
  while (BN > 4 && pa_smem(tile_rows, BN, H, G, D, E) > 200 * 1024) BN >>= 1;
  const size_t smem = pa_smem(tile_rows, BN, H, G, D, E);
  if (smem > 220 * 1024) return (int)cudaErrorInvalidValue;
  PoolAttnParams p{q, k_tok, v_tok, k_pool, v_pool, out, talk, tiles, q_start, q_len, seq_len, bt_tok, bt_pool,
                   bt_tok_stride, bt_pool_stride, H, G, D, E, page_tokens, window, pool, BN, scale,
                   split_tiles, splits, part_ml, stats, part_o, 0};
  if (dtype != PA_DTYPE) return (int)cudaErrorInvalidValue;
  switch (tile_rows) {
    case 1: return run_pa<PaT, 1>(p, n_tiles, smem, stream);
    case 4: return run_pa<PaT, 4>(p, n_tiles, smem, stream);
    case 16: return run_pa<PaT, 16>(p, n_tiles, smem, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}
