// Layer normalisation with weight and bias, fused with the residual sum on
// either side of it, and the embedding with a sinusoidal position vector.
//
//   LN(x) = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b
//
// A block that normalises a part's input AND its output ("sandwich") does, per
// token row, between two parts:
//
//   resid += LN_post(y)          y: the output of the part that just ran
//   h      = LN_pre(resid)       h: the input of the part that runs next
//
// `fb_ln_add_ln` makes both in one pass over the row; either half may be absent
// (the first norm of a model has no y, the last sum no h). Statistics, the sum
// and the residual are 32-bit; the variance is the mean of squared deviations
// taken in a second pass over the row held in shared memory.
//
// Between the two halves the stream may be replaced by a weighted sum over the
// streams that the layers so far have left (a depth-wise average):
//
//   X_n = resid (after the sum);   resid <- sum_j mix[j] X_j,  j = 0 .. n
//
// X_0 is `first` (the stream as the embedding left it), X_1 .. X_n are the rows
// of `kept` ([n, T, W]; X_n is written here), and the terms are added in the
// order of j.
#include "common.cuh"

namespace {

struct DepthMix {
  const float* first;    // X_0 [T, W]
  float* kept;           // X_1 .. X_n, [n, T, W]
  const float* weights;  // [n + 1] on the device
  int n;                 // 0: no mixing
  long long plane;       // T * W
};

// row[] holds the residual row after its sum; keeps it as X_n and replaces it (in
// shared memory and in `x`) by the weighted sum over X_0 .. X_n.
__device__ __forceinline__ void depth_mix_row(const DepthMix& m, float* row, float* x, size_t base,
                                              int W) {
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float last = row[i];
    m.kept[(size_t)(m.n - 1) * m.plane + base + i] = last;
    float v = m.weights[0] * __ldcg(m.first + base + i);
    for (int j = 1; j < m.n; ++j)
      v = fmaf(m.weights[j], __ldcg(m.kept + (size_t)(j - 1) * m.plane + base + i), v);
    v = fmaf(m.weights[m.n], last, v);
    x[i] = v;
    row[i] = v;
  }
  __syncthreads();
}

template <typename TY, typename TO>
__global__ void ln_add_ln_kernel(const TY* y, const float* __restrict__ w1,
                                 const float* __restrict__ b1, float y_scale, float* resid,
                                 const float* __restrict__ w2, const float* __restrict__ b2,
                                 TO* __restrict__ out, int W, float eps, float inv_w,
                                 DepthMix mix) {
  fb_pdl_launch();
  fb_pdl_wait();
  extern __shared__ float row[];  // W floats
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * W;
  float* x = resid + base;
  if (y != nullptr && w1 == nullptr) {  // a plain sum: y joins the residual times a constant
    const TY* yr = y + base;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = fmaf(y_scale, fb_load_coherent<TY>(yr + i), x[i]);
      x[i] = v;
      row[i] = v;
    }
  } else if (y != nullptr) {
    const TY* yr = y + base;
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = fb_load_coherent<TY>(yr + i);
      row[i] = v;
      s += v;
    }
    const float mean = fb_block_sum(s, scratch) * inv_w;
    float q = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float d = row[i] - mean;
      q += d * d;
    }
    const float r = 1.0f / sqrtf(fb_block_sum(q, scratch) * inv_w + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = x[i] + ((row[i] - mean) * r * w1[i] + b1[i]);
      x[i] = v;
      row[i] = v;
    }
  } else if (out != nullptr || mix.n > 0) {
    for (int i = threadIdx.x; i < W; i += blockDim.x) row[i] = x[i];
  }
  if (mix.n > 0) depth_mix_row(mix, row, x, base, W);
  if (out == nullptr) return;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += row[i];
  const float mean = fb_block_sum(s, scratch) * inv_w;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float d = row[i] - mean;
    q += d * d;
  }
  const float r = 1.0f / sqrtf(fb_block_sum(q, scratch) * inv_w + eps);
  TO* o = out + base;
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    o[i] = fb_from_float<TO>((row[i] - mean) * r * w2[i] + (b2 != nullptr ? b2[i] : 0.f));
}

// The same for rows of whole groups of four elements on 16-byte boundaries: every
// global and shared access is a float4 (or four 16-bit values in one 8-byte piece).
template <typename TD>
__device__ __forceinline__ float4 ld4(const TD* p);
template <>
__device__ __forceinline__ float4 ld4<float>(const float* p) {
  return __ldcg(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename TD>
__device__ __forceinline__ void st4(TD* p, float4 v);
template <>
__device__ __forceinline__ void st4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TY, typename TO>
__global__ void ln_add_ln_vec_kernel(const TY* y, const float* __restrict__ w1,
                                     const float* __restrict__ b1, float y_scale, float* resid,
                                     const float* __restrict__ w2, const float* __restrict__ b2,
                                     TO* __restrict__ out, int W, float eps, float inv_w,
                                     DepthMix mix) {
  fb_pdl_launch();
  fb_pdl_wait();
  extern __shared__ __align__(16) float row[];  // W floats
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * W;
  float* x = resid + base;
  float4* row4 = reinterpret_cast<float4*>(row);
  const int n4 = W / 4;
  if (y != nullptr && w1 == nullptr) {
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 a = ld4<float>(x + 4 * i), d = ld4<TY>(y + base + 4 * i);
      const float4 v = make_float4(fmaf(y_scale, d.x, a.x), fmaf(y_scale, d.y, a.y),
                                   fmaf(y_scale, d.z, a.z), fmaf(y_scale, d.w, a.w));
      st4<float>(x + 4 * i, v);
      row4[i] = v;
    }
  } else if (y != nullptr) {
    float s = 0.f;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 v = ld4<TY>(y + base + 4 * i);
      row4[i] = v;
      s += (v.x + v.y) + (v.z + v.w);
    }
    const float mean = fb_block_sum(s, scratch) * inv_w;
    float q = 0.f;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 v = row4[i];
      const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
      q += (a * a + b * b) + (c * c + d * d);
    }
    const float r = 1.0f / sqrtf(fb_block_sum(q, scratch) * inv_w + eps);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 v = row4[i], g = ld4<float>(w1 + 4 * i), h = ld4<float>(b1 + 4 * i);
      const float4 a = ld4<float>(x + 4 * i);
      const float4 o = make_float4(a.x + ((v.x - mean) * r * g.x + h.x), a.y + ((v.y - mean) * r * g.y + h.y),
                                   a.z + ((v.z - mean) * r * g.z + h.z), a.w + ((v.w - mean) * r * g.w + h.w));
      st4<float>(x + 4 * i, o);
      row4[i] = o;
    }
  } else if (out != nullptr || mix.n > 0) {
    for (int i = threadIdx.x; i < n4; i += blockDim.x) row4[i] = ld4<float>(x + 4 * i);
  }
  if (mix.n > 0) depth_mix_row(mix, row, x, base, W);
  if (out == nullptr) return;
  float s = 0.f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = row4[i];
    s += (v.x + v.y) + (v.z + v.w);
  }
  const float mean = fb_block_sum(s, scratch) * inv_w;
  float q = 0.f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = row4[i];
    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
    q += (a * a + b * b) + (c * c + d * d);
  }
  const float r = 1.0f / sqrtf(fb_block_sum(q, scratch) * inv_w + eps);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = row4[i], g = ld4<float>(w2 + 4 * i);
    const float4 h = b2 != nullptr ? ld4<float>(b2 + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    st4<TO>(out + base + 4 * i, make_float4((v.x - mean) * r * g.x + h.x, (v.y - mean) * r * g.y + h.y,
                                            (v.z - mean) * r * g.z + h.z, (v.w - mean) * r * g.w + h.w));
  }
}

// x[t, :] = table[ids[t], :] * scale + pe(positions[t]), pe[2i] = sin(p f_i),
// pe[2i+1] = cos(p f_i). The angle is the double-precision product of the
// position and a double-precision frequency, so that it is exact to 32 bits
// at any position; `copy`, when given, receives the same rows.
template <typename T>
__global__ void embed_sinusoid_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                      const int* __restrict__ positions,
                                      const double* __restrict__ freq, float scale,
                                      float* __restrict__ out, float* __restrict__ copy, int W,
                                      int V) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const double p = (double)positions[t];
  const bool inside = id >= 0 && id < V;
  const T* src = table + (size_t)(inside ? id : 0) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const double angle = p * freq[i >> 1];
    const float pe = (float)((i & 1) ? cos(angle) : sin(angle));
    const float e = inside ? fb_to_float<T>(src[i]) * scale : 0.f;
    const float v = e + pe;
    out[(size_t)t * W + i] = v;
    if (copy != nullptr) copy[(size_t)t * W + i] = v;
  }
}

// out[t, :W] = resid[t, :] (+ nothing), out[t, W:] = x0[t, :], rounded to the
// activation type: the input rows of a product over two streams side by side.
template <typename TO>
__global__ void concat_cast_kernel(const float* a, const float* b, TO* __restrict__ out, int W) {
  fb_pdl_launch();
  fb_pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    out[t * 2 * W + i] = fb_from_float<TO>(__ldcg(a + t * W + i));
    out[t * 2 * W + W + i] = fb_from_float<TO>(__ldcg(b + t * W + i));
  }
}

// x[t, :] += v[:]
__global__ void add_row_vector_kernel(float* x, const float* __restrict__ v, int W) {
  fb_pdl_launch();
  fb_pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) x[t * W + i] += v[i];
}
}  // namespace

FB_API int fb_ln_add_ln(const void* y, int y_dtype, const float* w1, const float* b1, float y_scale,
                        float* resid, const float* w2, const float* b2, void* out, int out_dtype,
                        int T, int W, float eps, const float* mix_first, float* mix_kept,
                        const float* mix_weights, int mix_n, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0 && eps > 0.f, "ln_add_ln: bad sizes T=%d W=%d", T, W);
  FB_REQUIRE(resid != nullptr, "ln_add_ln: no residual rows");
  FB_REQUIRE(y == nullptr || ((w1 != nullptr) == (b1 != nullptr)),
             "ln_add_ln: the norm of y has a weight or a bias but not both");
  FB_REQUIRE(out == nullptr || w2, "ln_add_ln: the norm of the sum has no weight");
  FB_REQUIRE(y_scale == 1.0f || w1 == nullptr, "ln_add_ln: a constant on y goes with a plain sum");
  FB_REQUIRE((size_t)W * 4 <= 200 * 1024, "ln_add_ln: rows of %d do not fit shared memory", W);
  FB_REQUIRE(mix_n >= 0 && (mix_n == 0 || (mix_first && mix_kept && mix_weights)),
             "ln_add_ln: a depth-wise average of %d kept streams lacks an input", mix_n);
  if (T == 0 || (y == nullptr && out == nullptr && mix_n == 0)) return 0;
  const DepthMix mix{mix_first, mix_kept, mix_weights, mix_n, (long long)T * W};
  const size_t smem = (size_t)W * 4;
  const bool vec = W % 4 == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)resid % 16) == 0 &&
                   ((uintptr_t)out % 16) == 0 && ((uintptr_t)w1 % 16) == 0 &&
                   ((uintptr_t)b1 % 16) == 0 && ((uintptr_t)w2 % 16) == 0 && ((uintptr_t)b2 % 16) == 0;
  // (the block width decides the order of a row's sums, so it depends on W alone)
  const int threads = vec ? (W >= 4096 ? 512 : (W >= 1024 ? 256 : 128))
                          : (W >= 2048 ? 512 : (W >= 512 ? 256 : 128));
#define FB_LN_LAUNCH(TY, TO)                                                                   \
  do {                                                                                         \
    static bool seen[64];                                                                      \
    if (smem > 48 * 1024 && fb_first_use_on_device(seen))                                      \
      cudaFuncSetAttribute(ln_add_ln_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           200 * 1024);                                                        \
    static bool seen_vec[64];                                                                  \
    if (smem > 48 * 1024 && fb_first_use_on_device(seen_vec))                                  \
      cudaFuncSetAttribute(ln_add_ln_vec_kernel<TY, TO>,                                       \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
    if (vec)                                                                                   \
      fb_launch(ln_add_ln_vec_kernel<TY, TO>, dim3(T), dim3(threads), smem, stream,            \
                (const TY*)y, w1, b1, y_scale, resid, w2, b2, (TO*)out, W, eps, 1.0f / (float)W,  \
                mix);                                                                          \
    else                                                                                       \
      fb_launch(ln_add_ln_kernel<TY, TO>, dim3(T), dim3(threads), smem, stream, (const TY*)y,  \
                w1, b1, y_scale, resid, w2, b2, (TO*)out, W, eps, 1.0f / (float)W, mix);       \
  } while (0)
  const int yd = y ? y_dtype : FB_F32, od = out ? out_dtype : FB_F32;
  FB_DISPATCH_DTYPE(yd, TY, FB_DISPATCH_DTYPE(od, TO, FB_LN_LAUNCH(TY, TO)));
#undef FB_LN_LAUNCH
  return fb_check_launch("ln_add_ln");
}

FB_API int fb_embed_sinusoid(const void* table, int table_dtype, const int* ids,
                             const int* positions, const double* freq, float scale, float* out,
                             float* copy, int T, int W, int V, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0 && W % 2 == 0 && V > 0, "embed_sinusoid: bad sizes T=%d W=%d V=%d", T,
             W, V);
  if (T == 0) return 0;
  const int threads = W >= 1024 ? 256 : 128;
  FB_DISPATCH_DTYPE(table_dtype, E, (fb_launch(embed_sinusoid_kernel<E>, dim3(T), dim3(threads), 0,
      stream, (const E*)table, ids, positions, freq, scale, out, copy, W, V)));
  return fb_check_launch("embed_sinusoid");
}

FB_API int fb_concat_cast(const float* a, const float* b, void* out, int out_dtype, int T, int W,
                          cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0, "concat_cast: bad sizes T=%d W=%d", T, W);
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(out_dtype, E, (fb_launch(concat_cast_kernel<E>, dim3(T), dim3(256), 0, stream,
      a, b, (E*)out, W)));
  return fb_check_launch("concat_cast");
}

FB_API int fb_add_row_vector(float* x, const float* v, int T, int W, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0, "add_row_vector: bad sizes T=%d W=%d", T, W);
  if (T == 0) return 0;
  fb_launch(add_row_vector_kernel, dim3(T), dim3(256), 0, stream, x, v, W);
  return fb_check_launch("add_row_vector");
}
