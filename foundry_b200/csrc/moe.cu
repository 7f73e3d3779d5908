// A feed-forward of routed experts.
//
//   z = W_router h (+ b) (32-bit). Two scoring rules (`score`):
//   0: the `top` experts of largest z are chosen (the lower index among equals);
//      their weights are the softmax over the chosen z only
//   1: s = sigmoid(z); the experts form `groups` equal groups of neighbours, a group's
//      score is the sum of its two largest s, only experts of the `keep` best groups can
//      be chosen (groups 1: all); the `top` largest s are chosen and weighted by s itself
//   y = sum_c weight_c * expert_c(h)
//   expert:  g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit)
//            a = g * sigmoid(alpha g) * (u + shift);  out = W_down a
//   (limit = infinity, alpha = 1, shift = 0: silu(g) * u)
//
// The experts' matrices are stacked: gate_up [E, 2 ff, W] (gate rows, then up
// rows) and down [E, W, ff]. `limit`, `alpha`, `shift` and the counts are parameters.
//
// `fb_moe_route` makes the choice per token. `fb_moe_experts_rows` is the form
// for a handful of tokens: one block per token streams the weights of that
// token's experts (each chosen expert's matrices once, 16-byte loads along K),
// with the hidden activations in shared memory and 32-bit sums throughout.
#include "common.cuh"

namespace {

// One token's choice, by one warp. s_all, s_group, s_plain: 256 floats each of this warp's own.
__device__ __forceinline__ void route_token(const float* z, long long ld,
                                            const float* __restrict__ bias, int E, int top,
                                            int* __restrict__ chosen, float* __restrict__ weights,
                                            int score, int groups, int keep,
                                            const float* __restrict__ correction, int normalise,
                                            float sum_floor, float weight_scale, int t, int lane,
                                            float* s_all, float* s_group, float* s_plain) {
  // each lane keeps the experts lane, lane + 32, ... (up to 8 of them).
  // v[] is what the choice goes by (the score, plus `correction` where given); the
  // weights come from the scores themselves (s_plain).
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    v[i] = -INFINITY;
    if (e < E) {
      const float x = __ldcg(z + (size_t)t * ld + e) + (bias != nullptr ? bias[e] : 0.f);
      const float sc = score == 1 ? 1.0f / (1.0f + expf(-x)) : x;
      s_plain[e] = sc;
      v[i] = correction != nullptr ? sc + correction[e] : sc;
    }
  }
  __syncwarp();
  if (score == 1 && groups > 1) {
    // a group's score: the sum of its two largest (a group of one: that one); the `keep`
    // best groups stay, the lower index among equals
    const int per = E / groups;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (lane + 32 * i < E) s_all[lane + 32 * i] = v[i];
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;
      for (int k = 0; k < per; ++k) {
        const float x = s_all[g * per + k];
        if (x > a) { b = a; a = x; } else if (x > b) { b = x; }
      }
      s_group[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    for (int c = 0; c < keep; ++c) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)  // (a group kept earlier is marked with INFINITY)
        if (s_group[g] != INFINITY && s_group[g] > best) { best = s_group[g]; at = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      __syncwarp();
      if (lane == 0 && at < groups) s_group[at] = INFINITY;  // kept (a sum of scores is finite)
      __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      if (e < E && s_group[e / per] != INFINITY) v[i] = -INFINITY;
    }
  }
  float first = 0.f, sum = 0.f, mine = 0.f;
  for (int c = 0; c < top; ++c) {  // top <= 32: lane c keeps the c-th chosen value
    float best = -INFINITY;
    int at = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v[i] > best) { best = v[i]; at = lane + 32 * i; }
    // the largest value, and among equals the lowest index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (c == 0) first = best;  // values are chosen in falling order: the first is the largest
    if (at >= E) at = 0;  // only when every value left is NaN: any expert, never a wild index
    const float e = score == 1 ? s_plain[at] : expf(best - first);
    sum += e;
    if (lane == c) mine = e;
    if (lane == 0) chosen[(size_t)t * top + c] = at;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (at == lane + 32 * i) v[i] = -INFINITY;
  }
  // sigmoid scores: the chosen scores themselves, or (normalise) their shares of their sum
  // plus `sum_floor`; both times `weight_scale`. Softmax over the chosen: mine / sum.
  if (lane < top)
    weights[(size_t)t * top + lane] =
        score == 1 ? (normalise ? mine / (sum + sum_floor) * weight_scale : mine * weight_scale)
                   : mine / sum;
  __syncwarp();  // a warp that goes on to another token writes the shared tables again
}

__global__ void moe_route_kernel(const float* z, long long ld, const float* __restrict__ bias,
                                 int E, int top, int* __restrict__ chosen,
                                 float* __restrict__ weights, int score, int groups, int keep,
                                 const float* __restrict__ correction, int normalise,
                                 float sum_floor, float weight_scale) {
  fb_pdl_launch();
  fb_pdl_wait();
  // one warp per token
  __shared__ float s_all[256];
  __shared__ float s_group[256];
  __shared__ float s_plain[256];
  route_token(z, ld, bias, E, top, chosen, weights, score, groups, keep, correction, normalise,
              sum_floor, weight_scale, blockIdx.x, threadIdx.x & 31, s_all, s_group, s_plain);
}

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* x, int K, int lane);
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ w, const float* x, int K,
                                                int lane) {
  float acc = 0.f;
  for (int k = lane; k < K; k += 32) acc = fmaf(w[k], x[k], acc);
  return fb_warp_sum(acc);
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w,
                                                        const float* x, int K, int lane) {
  float acc = 0.f;
  if (K % 8 == 0 && ((uintptr_t)w % 16) == 0) {
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + k);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc = fmaf(f.x, x[k + 2 * i], acc);
        acc = fmaf(f.y, x[k + 2 * i + 1], acc);
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(w[k]), x[k], acc);
  }
  return fb_warp_sum(acc);
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_experts_rows_kernel(const T* h, const T* __restrict__ gate_up, const T* __restrict__ down,
                        const int* chosen, const float* weights, float* __restrict__ out, int W,
                        int ff, int top, int E, float limit, float alpha, float shift,
                        const float* addend) {
  fb_pdl_wait();
  extern __shared__ float smem[];  // x [W] | act [ff] | acc [W]
  float* x = smem;
  float* act = smem + W;
  float* acc = act + ff;
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    x[i] = fb_load_coherent<T>(h + (size_t)t * W + i);
    acc[i] = 0.f;
  }
  __syncthreads();
  for (int c = 0; c < top; ++c) {
    const int e = __ldcg(chosen + (size_t)t * top + c);
    if (e < 0 || e >= E) continue;  // uniform over the block
    const float wt = __ldcg(weights + (size_t)t * top + c);
    const T* gu = gate_up + (size_t)e * 2 * ff * W;
    for (int f = warp; f < ff; f += nwarps) {
      float g = dot_row<T>(gu + (size_t)f * W, x, W, lane);
      float u = dot_row<T>(gu + (size_t)(ff + f) * W, x, W, lane);
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      if (lane == 0) act[f] = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift);
    }
    __syncthreads();
    const T* dn = down + (size_t)e * W * ff;
    for (int r = warp; r < W; r += nwarps) {
      const float y = dot_row<T>(dn + (size_t)r * ff, act, ff, lane);
      if (lane == 0) acc[r] = fmaf(wt, y, acc[r]);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[(size_t)t * W + i] =
        acc[i] + (addend != nullptr ? __ldcg(addend + (size_t)t * W + i) : 0.f);
}
}  // namespace

FB_API int fb_moe_route(const float* z, long long ld, const float* bias, int E, int top,
                        int* chosen, float* weights, int T, int score, int groups, int keep,
                        const float* correction, int normalise, float sum_floor,
                        float weight_scale, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && E > 0 && E <= 256 && top > 0 && top <= E && top <= 32 && ld >= E,
             "moe_route: %d experts (at most 256), %d chosen (at most 32)", E, top);
  FB_REQUIRE(score == 0 || score == 1, "moe_route: unknown scoring rule %d", score);
  FB_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups &&
             (long long)keep * (E / groups) >= top,
             "moe_route: %d groups of %d experts, %d kept, %d chosen", groups, E, keep, top);
  FB_REQUIRE(score == 1 || groups == 1, "moe_route: groups need the sigmoid scores");
  FB_REQUIRE(score == 1 || (correction == nullptr && !normalise && weight_scale == 1.0f),
             "moe_route: a correction of the choice, shares of the sum and a constant on the "
             "weights need the sigmoid scores");
  if (T == 0) return 0;
  // a warp per token
  fb_launch(moe_route_kernel, dim3(T), dim3(32), 0, stream, z, ld, bias, E, top, chosen, weights,
            score, groups, keep, correction, normalise, sum_floor, weight_scale);
  return fb_check_launch("moe_route");
}

FB_API int fb_moe_experts_rows(const void* h, int dtype, const void* gate_up, const void* down,
                               const int* chosen, const float* weights, float* out, int T, int W,
                               int ff, int top, int E, float limit, float alpha, float shift,
                               const float* addend, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0 && ff > 0 && top > 0, "moe_experts_rows: bad sizes");
  const size_t smem = (size_t)(2 * W + ff) * 4;
  FB_REQUIRE(smem <= 200 * 1024, "moe_experts_rows: width %d and %d hidden units do not fit "
             "shared memory", W, ff);
  if (T == 0) return 0;
#define FB_MOE_ROWS(E_)                                                                         \
  do {                                                                                          \
    static bool seen[64];                                                                       \
    if (smem > 48 * 1024 && fb_first_use_on_device(seen))                                       \
      cudaFuncSetAttribute(moe_experts_rows_kernel<E_>,                                         \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);            \
    fb_launch(moe_experts_rows_kernel<E_>, dim3(T), dim3(256), smem, stream, (const E_*)h,      \
              (const E_*)gate_up, (const E_*)down, chosen, weights, out, W, ff, top, E, limit,  \
              alpha, shift, addend);                                                            \
  } while (0)
  FB_DISPATCH_DTYPE(dtype, E_, FB_MOE_ROWS(E_));
#undef FB_MOE_ROWS
  return fb_check_launch("moe_experts_rows");
}

// ===================================================================== grouped
// Many (token, choice) pairs: pairs are sorted by expert on the device, so that
// an expert's matrices are read once for all of its tokens.
//
//   fb_moe_sort       counts per expert, their running sums, and for every pair
//                     its place in the expert-sorted order (`place[t * top + c]`)
//                     with the inverse list `pair_at[place]`
//   fb_moe_gather     x_sorted[place] = x[token of the pair]
//   fb_moe_gate_up_grouped / fb_moe_down_grouped
//                     the two products for a handful of tokens per expert: a
//                     block owns (expert, a slice of weight rows), stages up to
//                     CHUNK of the expert's input rows in shared memory and
//                     streams its weight rows once per chunk (CUDA cores,
//                     32-bit sums); the activation is the first one's epilogue
//   fb_moe_glu        the activation alone, for products made elsewhere
//   fb_moe_combine    out[t] = sum_c weight[t, c] * y_sorted[place[t, c]] in the
//                     order of c, so the sum does not depend on the sorting
namespace {

__device__ __forceinline__ void sort_pairs(const int* chosen, int n_pairs, int E,
                                           int* __restrict__ counts, int* __restrict__ starts,
                                           int* __restrict__ place, int* __restrict__ pair_at) {
  // one block; counts and starts live in shared memory (E <= 256)
  __shared__ int cnt[256], start[257];
  for (int e = threadIdx.x; e < 256; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) { start[e] = at; at += cnt[e]; }
    start[E] = at;
  }
  __syncthreads();
  // a warp places the pairs of an expert in the order of their indices (a fixed
  // order): 32 pairs at a time, each lane's place from a ballot of the matching lanes
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    int at = start[e];
    for (int base = 0; base < n_pairs; base += 32) {
      const int i = base + lane;
      const bool mine = i < n_pairs && chosen[i] == e;
      const unsigned hits = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int where = at + __popc(hits & ((1u << lane) - 1u));
        place[i] = where;
        pair_at[where] = i;
      }
      at += __popc(hits);
    }
    if (lane == 0) { counts[e] = cnt[e]; starts[e] = start[e]; }
  }
  if (threadIdx.x == 0) starts[E] = start[E];
  // pairs without a valid expert (never for finite logits) are put nowhere
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e < 0 || e >= E) place[i] = -1;
  }
}

__global__ void moe_sort_kernel(const int* chosen, int n_pairs, int E, int* __restrict__ counts,
                                int* __restrict__ starts, int* __restrict__ place,
                                int* __restrict__ pair_at) {
  fb_pdl_wait();
  sort_pairs(chosen, n_pairs, E, counts, starts, place, pair_at);
}

// Choice and sort in one block, for the few tokens of a single-token step: eight warps
// take the tokens in turn, then the block sorts the pairs it has just written.
constexpr int ROUTE_SORT_WARPS = 8;
__global__ void __launch_bounds__(ROUTE_SORT_WARPS * 32)
moe_route_sort_kernel(const float* z, long long ld, const float* __restrict__ bias, int E, int top,
                      int* chosen, float* __restrict__ weights, int score, int groups, int keep,
                      const float* __restrict__ correction, int normalise, float sum_floor,
                      float weight_scale, int T, int* __restrict__ counts,
                      int* __restrict__ starts, int* __restrict__ place,
                      int* __restrict__ pair_at) {
  fb_pdl_launch();
  fb_pdl_wait();
  __shared__ float s_all[ROUTE_SORT_WARPS][256];
  __shared__ float s_group[ROUTE_SORT_WARPS][256];
  __shared__ float s_plain[ROUTE_SORT_WARPS][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = warp; t < T; t += ROUTE_SORT_WARPS)
    route_token(z, ld, bias, E, top, chosen, weights, score, groups, keep, correction, normalise,
                sum_floor, weight_scale, t, lane, s_all[warp], s_group[warp], s_plain[warp]);
  __syncthreads();  // the block's own writes of `chosen` are visible to all its threads
  sort_pairs(chosen, T * top, E, counts, starts, place, pair_at);
}

template <typename T>
__global__ void moe_gather_kernel(const T* x, const int* pair_at, const int* starts, int E, int top,
                                  T* __restrict__ out, int W) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int at = blockIdx.x;
  if (at >= starts[E]) return;
  const int t = pair_at[at] / top;
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)at * W + i] = x[(size_t)t * W + i];
}

__device__ __forceinline__ float glu_act(float g, float u, float limit, float alpha, float shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift);
}

template <typename TI, typename TO>
__global__ void moe_glu_kernel(const TI* gu, TO* __restrict__ out, int ff, float limit, float alpha, float shift,
                               const int* starts, int E) {
  fb_pdl_launch();
  fb_pdl_wait();
  const size_t row = blockIdx.x;
  if ((int)row >= starts[E]) return;
  for (int f = threadIdx.x; f < ff; f += blockDim.x)
    out[row * ff + f] = fb_from_float<TO>(glu_act(fb_load_coherent<TI>(gu + row * 2 * ff + f),
                                                  fb_load_coherent<TI>(gu + row * 2 * ff + ff + f),
                                                  limit, alpha, shift));
}

// 8 consecutive weights of a row as floats
template <typename T>
__device__ __forceinline__ void w8(const T* __restrict__ p, float (&v)[8]);
template <>
__device__ __forceinline__ void w8<float>(const float* __restrict__ p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void w8<__nv_bfloat16>(const __nv_bfloat16* __restrict__ p,
                                                  float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// A block owns (expert e, weight rows [row0, row0 + rows)); K % 8 == 0 and the
// weight rows 16-byte aligned (checked by the launcher). NR weight rows are
// walked together by a warp: GATED walks a gate row and its up row (NR = 2).
// xs: the chunk's input rows [CHUNK][K] as floats in shared memory. (A form with two
// rows a chunk for single-token steps, four blocks a SM, was slower: 141 against
// 103 us a call at 16 pairs over 16 experts of 2048 x 2048.)
// `pair_at` given: the sorted row `at` is row pair_at[at] / top of x (no gathered copy).
template <typename T, typename TX, bool GATED, int CHUNK>
__global__ void __launch_bounds__(256, 2)
moe_grouped_kernel(const TX* x, long long ldx, const T* __restrict__ w, const int* starts,
                   float* __restrict__ out, long long ldo, int K, int N, int rows_per_block,
                   float limit, float alpha, float shift, const int* pair_at, int top) {
  fb_pdl_wait();
  extern __shared__ float xs[];  // [CHUNK][K]
  const int e = blockIdx.x;
  const int begin = starts[e], end = starts[e + 1];
  if (begin >= end) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(N, row0 + rows_per_block);
  // GATED: w is [E][2N][K] (gate rows, then up rows), else [E][N][K]
  const T* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
  for (int c0 = begin; c0 < end; c0 += CHUNK) {
    const int nc = min(CHUNK, end - c0);
    __syncthreads();
    for (int i = threadIdx.x; i < nc * K; i += blockDim.x) {
      const int r = i / K, k = i - r * K;
      const size_t src = pair_at != nullptr ? (size_t)(pair_at[c0 + r] / top) : (size_t)(c0 + r);
      xs[r * K + k] = fb_load_coherent<TX>(x + src * ldx + k);
    }
    __syncthreads();
    for (int row = row0 + warp; row < row1; row += nwarps) {
      float acc[CHUNK], acc2[CHUNK];
#pragma unroll
      for (int r = 0; r < CHUNK; ++r) acc[r] = acc2[r] = 0.f;
      const T* wr = we + (size_t)row * K;
      const T* wr2 = we + (size_t)(N + row) * K;
      // two steps of 256 weights at a time, read one round ahead: the loads of the next
      // 512 weights are on their way while the sums over these are made
      float an[2][8], bn[2][8];
      auto fetch = [&](int k0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (k0 + u * 256 < K) {
            w8<T>(wr + k0 + u * 256, an[u]);
            if (GATED) w8<T>(wr2 + k0 + u * 256, bn[u]);
          }
        }
      };
      fetch(lane * 8);
      for (int k0 = lane * 8; k0 < K; k0 += 512) {
        float a[2][8], b[2][8];
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[u][e] = an[u][e]; if (GATED) b[u][e] = bn[u][e]; }
        if (k0 + 512 < K) fetch(k0 + 512);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int k = k0 + u * 256;
          if (k < K) {
#pragma unroll
            for (int r = 0; r < CHUNK; ++r) {
              if (r < nc) {
                const float4 x0 = *reinterpret_cast<const float4*>(xs + r * K + k);
                const float4 x1 = *reinterpret_cast<const float4*>(xs + r * K + k + 4);
                acc[r] = fmaf(a[u][0], x0.x, acc[r]); acc[r] = fmaf(a[u][1], x0.y, acc[r]);
                acc[r] = fmaf(a[u][2], x0.z, acc[r]); acc[r] = fmaf(a[u][3], x0.w, acc[r]);
                acc[r] = fmaf(a[u][4], x1.x, acc[r]); acc[r] = fmaf(a[u][5], x1.y, acc[r]);
                acc[r] = fmaf(a[u][6], x1.z, acc[r]); acc[r] = fmaf(a[u][7], x1.w, acc[r]);
                if (GATED) {
                  acc2[r] = fmaf(b[u][0], x0.x, acc2[r]); acc2[r] = fmaf(b[u][1], x0.y, acc2[r]);
                  acc2[r] = fmaf(b[u][2], x0.z, acc2[r]); acc2[r] = fmaf(b[u][3], x0.w, acc2[r]);
                  acc2[r] = fmaf(b[u][4], x1.x, acc2[r]); acc2[r] = fmaf(b[u][5], x1.y, acc2[r]);
                  acc2[r] = fmaf(b[u][6], x1.z, acc2[r]); acc2[r] = fmaf(b[u][7], x1.w, acc2[r]);
                }
              }
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < CHUNK; ++r) {
        if (r < nc) {  // uniform over the warp
          const float g = fb_warp_sum(acc[r]);
          const float u = GATED ? fb_warp_sum(acc2[r]) : 0.f;
          if (lane == 0)
            out[(size_t)(c0 + r) * ldo + row] = GATED ? glu_act(g, u, limit, alpha, shift) : g;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The same two products on the tensor cores (bfloat16, K a multiple of 64): up to 8
// input rows of an expert are the 8 columns of `mma.sync.m16n8k16`, 16 weight rows
// its rows. A warp owns a tile of 16 weight rows (GATED: the 16 gate rows and their 16
// up rows) and pulls the weights straight from global memory into A fragments: of a
// block of 64 weights a thread reads the 16 consecutive ones at 16 (lane % 4) of rows
// lane / 4 and lane / 4 + 8 (32 contiguous bytes a row), which it uses as its
// fragment elements of four k-steps. The dot product does not care in which order K
// is walked as long as the input rows are read in the same order, so the B fragment
// of k-step s is the four inputs at 16 (lane % 4) + 4 s of input row lane / 4, one
// 8-byte load from shared memory. The next block's weights are read while this
// block's four instructions run.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                               unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, "
               "{%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int MMA_ROWS = 8;   // input rows a chunk
constexpr int MMA_PAD = 4;    // elements between input rows in shared memory (bank spread)

template <bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_mma_kernel(const __nv_bfloat16* x, long long ldx, const __nv_bfloat16* __restrict__ w,
                       const int* starts, void* out, long long ldo, int K, int N, float limit,
                       float alpha, float shift, const int* pair_at, int top) {
  fb_pdl_wait();
  extern __shared__ __align__(16) __nv_bfloat16 xb[];  // [MMA_ROWS][K + MMA_PAD]
  const int e = blockIdx.x;
  const int begin = starts[e], end = starts[e + 1];
  if (begin >= end) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = (blockIdx.y * 8 + warp) * 16;
  const bool tile = row0 < N;
  const int ldxs = K + MMA_PAD;
  const __nv_bfloat16* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
  // rows past the matrix read its last row; their results are not stored
  const int ra = min(row0 + g, N - 1), rb = min(row0 + g + 8, N - 1);
  const uint4* ga = reinterpret_cast<const uint4*>(we + (size_t)ra * K + 16 * t);
  const uint4* gb = reinterpret_cast<const uint4*>(we + (size_t)rb * K + 16 * t);
  const uint4* ua = reinterpret_cast<const uint4*>(we + (size_t)(N + ra) * K + 16 * t);
  const uint4* ub = reinterpret_cast<const uint4*>(we + (size_t)(N + rb) * K + 16 * t);
  for (int c0 = begin; c0 < end; c0 += MMA_ROWS) {
    const int nc = min(MMA_ROWS, end - c0);
    __syncthreads();
    for (int i = threadIdx.x; i < MMA_ROWS * (K / 8); i += blockDim.x) {
      const int r = i / (K / 8), k = (i - r * (K / 8)) * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < nc) {
        const size_t src = pair_at != nullptr ? (size_t)(pair_at[c0 + r] / top) : (size_t)(c0 + r);
        v = __ldcg(reinterpret_cast<const uint4*>(x + src * ldx + k));
      }
      uint2* dst = reinterpret_cast<uint2*>(xb + (size_t)r * ldxs + k);  // rows are 8-byte aligned
      dst[0] = make_uint2(v.x, v.y);
      dst[1] = make_uint2(v.z, v.w);
    }
    __syncthreads();
    if (!tile) continue;
    float cg[4] = {0.f, 0.f, 0.f, 0.f}, cu[4] = {0.f, 0.f, 0.f, 0.f};
    const __nv_bfloat16* xrow = xb + (size_t)g * ldxs + 16 * t;
    uint4 na[2], nb[2], nua[2], nub[2];
    auto fetch = [&](int kb) {  // kb in units of 8 elements (a uint4)
      na[0] = __ldg(ga + kb); na[1] = __ldg(ga + kb + 1);
      nb[0] = __ldg(gb + kb); nb[1] = __ldg(gb + kb + 1);
      if (GATED) {
        nua[0] = __ldg(ua + kb); nua[1] = __ldg(ua + kb + 1);
        nub[0] = __ldg(ub + kb); nub[1] = __ldg(ub + kb + 1);
      }
    };
    fetch(0);
    for (int kb = 0; kb < K; kb += 64) {
      const unsigned a[8] = {na[0].x, na[0].y, na[0].z, na[0].w, na[1].x, na[1].y, na[1].z, na[1].w};
      const unsigned b[8] = {nb[0].x, nb[0].y, nb[0].z, nb[0].w, nb[1].x, nb[1].y, nb[1].z, nb[1].w};
      unsigned p[8], q[8];
      if (GATED) {
        p[0] = nua[0].x; p[1] = nua[0].y; p[2] = nua[0].z; p[3] = nua[0].w;
        p[4] = nua[1].x; p[5] = nua[1].y; p[6] = nua[1].z; p[7] = nua[1].w;
        q[0] = nub[0].x; q[1] = nub[0].y; q[2] = nub[0].z; q[3] = nub[0].w;
        q[4] = nub[1].x; q[5] = nub[1].y; q[6] = nub[1].z; q[7] = nub[1].w;
      }
      if (kb + 64 < K) fetch((kb + 64) / 8);
#pragma unroll
      for (int s2 = 0; s2 < 4; ++s2) {
        const uint2 xv = *reinterpret_cast<const uint2*>(xrow + kb + 4 * s2);
        mma_bf16_16816(cg, a[2 * s2], b[2 * s2], a[2 * s2 + 1], b[2 * s2 + 1], xv.x, xv.y);
        if (GATED) mma_bf16_16816(cu, p[2 * s2], q[2 * s2], p[2 * s2 + 1], q[2 * s2 + 1], xv.x, xv.y);
      }
    }
    // c[0], c[1]: weight row g, input rows 2t and 2t + 1; c[2], c[3]: weight row g + 8
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = row0 + g + (i >> 1) * 8, n = 2 * t + (i & 1);
      if (row < N && n < nc) {
        if (GATED)
          reinterpret_cast<__nv_bfloat16*>(out)[(size_t)(c0 + n) * ldo + row] =
              __float2bfloat16_rn(glu_act(cg[i], cu[i], limit, alpha, shift));
        else
          reinterpret_cast<float*>(out)[(size_t)(c0 + n) * ldo + row] = cg[i];
      }
    }
  }
}

// out[t] = sum_c weights[t, c] * y[place[t, c]] (+ addend[t], what every token gets
// beside its experts: a shared expert's rows)
__global__ void moe_combine_kernel(const float* y, const int* place, const float* weights, int top,
                                   float* __restrict__ out, int W, const float* addend) {
  fb_pdl_launch();
  fb_pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < W; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int c = 0; c < top; ++c) {
      const int at = place[t * top + c];
      if (at >= 0) acc = fmaf(weights[t * top + c], __ldcg(y + (size_t)at * W + i), acc);
    }
    if (addend != nullptr) acc += __ldcg(addend + t * W + i);
    out[t * W + i] = acc;
  }
}
}  // namespace

FB_API int fb_moe_sort(const int* chosen, int n_pairs, int E, int* counts, int* starts, int* place,
                       int* pair_at, cudaStream_t stream) {
  FB_REQUIRE(n_pairs >= 0 && E > 0 && E <= 256, "moe_sort: %d experts (at most 256)", E);
  fb_launch(moe_sort_kernel, dim3(1), dim3(256), 0, stream, chosen, n_pairs, E, counts, starts,
            place, pair_at);
  return fb_check_launch("moe_sort");
}

// fb_moe_route and fb_moe_sort as one launch of one block (for up to a few dozen tokens).
FB_API int fb_moe_route_sort(const float* z, long long ld, const float* bias, int E, int top,
                             int* chosen, float* weights, int T, int score, int groups, int keep,
                             const float* correction, int normalise, float sum_floor,
                             float weight_scale, int* counts, int* starts, int* place,
                             int* pair_at, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && E > 0 && E <= 256 && top > 0 && top <= E && top <= 32 && ld >= E,
             "moe_route_sort: %d experts (at most 256), %d chosen (at most 32)", E, top);
  FB_REQUIRE(score == 0 || score == 1, "moe_route_sort: unknown scoring rule %d", score);
  FB_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups &&
             (long long)keep * (E / groups) >= top,
             "moe_route_sort: %d groups of %d experts, %d kept, %d chosen", groups, E, keep, top);
  FB_REQUIRE(score == 1 || (groups == 1 && correction == nullptr && !normalise &&
                            weight_scale == 1.0f),
             "moe_route_sort: groups, a correction, shares of the sum and a constant on the "
             "weights need the sigmoid scores");
  fb_launch(moe_route_sort_kernel, dim3(1), dim3(ROUTE_SORT_WARPS * 32), 0, stream, z, ld, bias, E,
            top, chosen, weights, score, groups, keep, correction, normalise, sum_floor,
            weight_scale, T, counts, starts, place, pair_at);
  return fb_check_launch("moe_route_sort");
}

FB_API int fb_moe_gather(const void* x, int dtype, const int* pair_at, const int* starts, int E,
                         int top, void* out, int n_pairs, int W, cudaStream_t stream) {
  FB_REQUIRE(n_pairs >= 0 && W > 0 && top > 0, "moe_gather: bad sizes");
  if (n_pairs == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, T_, (fb_launch(moe_gather_kernel<T_>, dim3(n_pairs), dim3(256), 0,
      stream, (const T_*)x, pair_at, starts, E, top, (T_*)out, W)));
  return fb_check_launch("moe_gather");
}

FB_API int fb_moe_glu(const void* gu, int in_dtype, void* out, int out_dtype, int n_pairs, int ff,
                      float limit, float alpha, float shift, const int* starts, int E, cudaStream_t stream) {
  FB_REQUIRE(n_pairs >= 0 && ff > 0, "moe_glu: bad sizes");
  if (n_pairs == 0) return 0;
  FB_DISPATCH_DTYPE(in_dtype, TI, FB_DISPATCH_DTYPE(out_dtype, TO, (fb_launch(
      moe_glu_kernel<TI, TO>, dim3(n_pairs), dim3(256), 0, stream, (const TI*)gu, (TO*)out, ff,
      limit, alpha, shift, starts, E))));
  return fb_check_launch("moe_glu");
}

// gated = 1: x rows in the weights' element type, w = gate_up [E, 2N, K], out = activations
// gated = 0: x rows are float32 (the activations), w = down [E, N, K], out = products
FB_API int fb_moe_grouped(int gated, const void* x, long long ldx, const void* w, int w_dtype,
                          const int* starts, float* out, long long ldo, int E, int K, int N,
                          float limit, float alpha, float shift, int sm_count, const int* pair_at, int top,
                          int n_pairs, cudaStream_t stream) {
  FB_REQUIRE(E > 0 && K > 0 && N > 0 && ldx >= K && ldo >= N, "moe_grouped: bad sizes");
  FB_REQUIRE(K % 8 == 0 && ((uintptr_t)w % 16) == 0 && ldx % 4 == 0,
             "moe_grouped: K = %d must be a multiple of 8 and the matrices 16-byte aligned", K);
  const int chunk = 8;
  const size_t smem = (size_t)chunk * K * 4;
  FB_REQUIRE(smem <= 200 * 1024, "moe_grouped: %d input rows of %d do not fit shared memory",
             chunk, K);
  FB_REQUIRE(pair_at == nullptr || top > 0, "moe_grouped: rows by pair need the pairs a token");
  // row slices so that the experts in use cover the SMs a few times over
  int slices = (6 * (sm_count > 0 ? sm_count : 148) + E - 1) / E;
  int rows = (N + slices - 1) / slices;
  rows = (rows + 7) / 8 * 8;
  dim3 grid(E, (N + rows - 1) / rows);
#define FB_MOE_GROUPED_C(T_, TX_, G_, C_)                                                       \
  do {                                                                                          \
    static bool seen[64];                                                                       \
    if (fb_first_use_on_device(seen))                                                           \
      cudaFuncSetAttribute(moe_grouped_kernel<T_, TX_, G_, C_>,                                 \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);            \
    fb_launch(moe_grouped_kernel<T_, TX_, G_, C_>, grid, dim3(256), smem, stream,               \
              (const TX_*)x, ldx, (const T_*)w, starts, out, ldo, K, N, rows, limit, alpha, shift,     \
              pair_at, top);                                                                    \
  } while (0)
#define FB_MOE_GROUPED(T_, TX_, G_)                                                             \
  do {                                                                                          \
    FB_MOE_GROUPED_C(T_, TX_, G_, 8);                                                           \
  } while (0)
  if (gated) {
    FB_DISPATCH_DTYPE(w_dtype, T_, FB_MOE_GROUPED(T_, T_, true));
  } else {
    FB_DISPATCH_DTYPE(w_dtype, T_, FB_MOE_GROUPED(T_, float, false));
  }
#undef FB_MOE_GROUPED
#undef FB_MOE_GROUPED_C
  return fb_check_launch("moe_grouped");
}

// gated = 1: out is bfloat16 activations [pairs, N]; gated = 0: out is float32 [pairs, N].
FB_API int fb_moe_grouped_mma(int gated, const void* x, long long ldx, const void* w,
                              const int* starts, void* out, long long ldo, int E, int K, int N,
                              float limit, float alpha, float shift, const int* pair_at, int top,
                              cudaStream_t stream) {
  FB_REQUIRE(E > 0 && K > 0 && N > 0 && ldx >= K && ldo >= N, "moe_grouped_mma: bad sizes");
  FB_REQUIRE(K % 64 == 0 && ldx % 8 == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)x % 16) == 0,
             "moe_grouped_mma: K = %d must be a multiple of 64 and the rows 16-byte aligned", K);
  FB_REQUIRE(pair_at == nullptr || top > 0, "moe_grouped_mma: rows by pair need the pairs a token");
  const size_t smem = (size_t)MMA_ROWS * (K + MMA_PAD) * 2;
  FB_REQUIRE(smem <= 200 * 1024, "moe_grouped_mma: %d input rows of %d do not fit shared memory",
             MMA_ROWS, K);
  dim3 grid(E, (N + 127) / 128);
  if (gated) {
    static bool seen[64];
    if (fb_first_use_on_device(seen))
      cudaFuncSetAttribute(moe_grouped_mma_kernel<true>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    fb_launch(moe_grouped_mma_kernel<true>, grid, dim3(256), smem, stream,
              (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, starts, out, ldo, K, N, limit,
              alpha, shift, pair_at, top);
  } else {
    static bool seen[64];
    if (fb_first_use_on_device(seen))
      cudaFuncSetAttribute(moe_grouped_mma_kernel<false>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    fb_launch(moe_grouped_mma_kernel<false>, grid, dim3(256), smem, stream,
              (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, starts, out, ldo, K, N, limit,
              alpha, shift, pair_at, top);
  }
  return fb_check_launch("moe_grouped_mma");
}

FB_API int fb_moe_combine(const float* y, const int* place, const float* weights, int top,
                          float* out, int T, int W, const float* addend, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0 && top > 0, "moe_combine: bad sizes");
  if (T == 0) return 0;
  const int want = (W + 255) / 256;  // few tokens: a row's columns go to several blocks
  const int parts = T <= 256 ? (want < 32 ? want : 32) : 1;
  fb_launch(moe_combine_kernel, dim3(T, parts), dim3(256), 0, stream, y, place, weights, top, out, W,
            addend);
  return fb_check_launch("moe_combine");
}
