// Mixers that carry a state of fixed size from token to token: the pieces
// around two linear recurrences over a per-head matrix state S [dim, vdim].
//
// Gated delta rule with a decay per key channel, or one decay a head (one step, per head):
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// RWKV-style time mixing with a bonus for the current token (per head):
//   o = (S + diag(b) k v^T)^T r;  S <- diag(w) S + k v^T
// State-space duality (Mamba-2) with one decay a head, a step size and a skip (per head):
//   S <- g S + k (step v)^T;  o = S^T q + skip v
//
// Both recurrences act on the columns of S independently, so a thread owns a
// slice of one column in registers (16 consecutive key rows at most, a column
// shared by KP lanes) and columns are spread over lanes, warps and blocks. A step
// is two dot products over the key rows, finished by shuffles among the KP
// lanes of a column. The state is 32-bit and lives in the sequence's state row
// between steps; every sequence of the step is walked by its own blocks from
// `cu_tokens`, so a step may bring any number of tokens per sequence.
//
// Around them, per token: the mix with the previous token's input (token
// shift), a short causal convolution with SiLU and unit-length heads, the
// decays, and the per-head RMS norm with an output gate. The inputs that these
// need from before the step (the previous token's row, the convolution's last
// taps - 1 inputs) are part of the state row too, written by
// `fb_state_tail_update` after their readers have run.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------- token shift
// out[m, t, :] = h[t] + (h[t-1] - h[t]) * mu[m], h[t-1] being the state's row
// for the first token that a sequence brings in this step.
template <typename T>
__global__ void token_shift_mix_kernel(const T* h, float* state, long long state_stride,
                                       long long prev_offset, const float* __restrict__ mu,
                                       T* __restrict__ out, const int* __restrict__ seq_of_token,
                                       const int* __restrict__ cu_tokens,
                                       const int* __restrict__ slots, int T_, int W, int n_mix,
                                       int single) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  if (seq < 0) {
    for (int m = 0; m < n_mix; ++m)
      for (int i = threadIdx.x; i < W; i += blockDim.x)
        out[((size_t)m * T_ + t) * W + i] = fb_from_float<T>(0.f);
    return;
  }
  const bool first = t == cu_tokens[seq];
  float* prev_state = state + (long long)slots[seq] * state_stride + prev_offset;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float x = fb_load_coherent<T>(h + (size_t)t * W + i);
    const float p = first ? __ldcg(prev_state + i) : fb_load_coherent<T>(h + (size_t)(t - 1) * W + i);
    const float d = p - x;
    for (int m = 0; m < n_mix; ++m)
      out[((size_t)m * T_ + t) * W + i] = fb_from_float<T>(x + d * mu[(size_t)m * W + i]);
    // `single`: every sequence of the step brings one token, so this block is the only
    // reader of the sequence's row and may leave the token's input there itself
    if (single) prev_state[i] = x;
  }
}

// ------------------------------------------------------- tail of the inputs
// state tail [n_tail, C] <- the last n_tail rows of (old tail ++ this step's rows).
template <typename T>
__global__ void state_tail_update_kernel(const T* x, long long ld, float* state,
                                         long long state_stride, long long offset, int n_tail,
                                         int C, const int* __restrict__ cu_tokens,
                                         const int* __restrict__ slots) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int seq = blockIdx.x;
  const int start = cu_tokens[seq], n = cu_tokens[seq + 1] - start;
  if (n <= 0) return;
  float* tail = state + (long long)slots[seq] * state_stride + offset;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    for (int r = 0; r < n_tail; ++r) {
      const int src = n + r;  // index into old tail (n_tail rows) followed by the step's rows
      const float v = src < n_tail ? tail[(size_t)src * C + c]
                                   : fb_load_coherent<T>(x + (size_t)(start + src - n_tail) * ld + c);
      tail[(size_t)r * C + c] = v;  // row r is read by no later iteration (src > r)
    }
  }
}

// ------------------------------------- causal convolution + SiLU + unit heads
// y[t, c] = silu(sum_a w[c, a] x[t - (taps - 1 - a), c] + bias[c]) (bias optional); rows in front of the
// step come from the state's tail, which holds zeros at a sequence's start.
// Then the first `n_unit` heads of `dim` channels are scaled to unit length,
// x / sqrt(sum(x^2) + unit_eps), the first `n_scaled` of them also by `extra`.
__global__ void conv_silu_unit_kernel(const float* x, long long ld, const float* __restrict__ w,
                                      const float* __restrict__ bias, int taps, float* state, long long state_stride,
                                      long long tail_offset, float* __restrict__ out, int C,
                                      const int* __restrict__ seq_of_token,
                                      const int* __restrict__ cu_tokens,
                                      const int* __restrict__ slots, int n_unit, int dim,
                                      int n_scaled, float extra, float unit_eps, int single) {
  fb_pdl_launch();
  fb_pdl_wait();
  extern __shared__ float y[];  // C floats
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  if (seq < 0) {
    for (int c = threadIdx.x; c < C; c += blockDim.x) out[(size_t)t * C + c] = 0.f;
    return;
  }
  const int start = cu_tokens[seq];
  const int n_tail = taps - 1;
  float* tail = state + (long long)slots[seq] * state_stride + tail_offset;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int a = 0; a < taps; ++a) {
      const int idx = t - (taps - 1 - a) - start;  // row of the step, negative: the tail
      const float v = idx >= 0 ? __ldcg(x + (size_t)(start + idx) * ld + c)
                               : __ldcg(tail + (size_t)(n_tail + idx) * C + c);
      acc = fmaf(w[(size_t)c * taps + a], v, acc);
      // `single` (one token a sequence: this block alone reads the row): the tail moves
      // on by one input as it is read, a thread touching only its own channel
      if (single && a > 0) tail[(size_t)(a - 1) * C + c] = v;
    }
    if (bias != nullptr) acc += bias[c];
    y[c] = acc * sigmoidf_(acc);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int head = warp; head < n_unit; head += nwarps) {
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss += y[head * dim + d] * y[head * dim + d];
    ss = fb_warp_sum(ss);
    const float r = (head < n_scaled ? extra : 1.0f) / sqrtf(ss + unit_eps);
    for (int d = lane; d < dim; d += 32) y[head * dim + d] *= r;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) out[(size_t)t * C + c] = y[c];
}

// The same without unit heads: nothing ties a token's channels together, so they are
// spread over blockIdx.y and written as they are made.
__global__ void conv_silu_kernel(const float* x, long long ld, const float* __restrict__ w,
                                 const float* __restrict__ bias, int taps, float* state,
                                 long long state_stride, long long tail_offset,
                                 float* __restrict__ out, int C, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                                 int single) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int seq = seq_of_token[t];
  if (seq < 0) {
    out[(size_t)t * C + c] = 0.f;
    return;
  }
  const int start = cu_tokens[seq];
  const int n_tail = taps - 1;
  float* tail = state + (long long)slots[seq] * state_stride + tail_offset;
  float acc = 0.f;
  for (int a = 0; a < taps; ++a) {
    const int idx = t - (taps - 1 - a) - start;  // row of the step, negative: the tail
    const float v = idx >= 0 ? __ldcg(x + (size_t)(start + idx) * ld + c)
                             : __ldcg(tail + (size_t)(n_tail + idx) * C + c);
    acc = fmaf(w[(size_t)c * taps + a], v, acc);
    if (single && a > 0) tail[(size_t)(a - 1) * C + c] = v;  // as in the kernel above
  }
  if (bias != nullptr) acc += bias[c];
  out[(size_t)t * C + c] = acc * sigmoidf_(acc);
}

// -------------------------------------------------------------------- decays
// mode 0: out <- exp(-exp(A[head]) * softplus(x + bias[c]))   (c = head * per_head + channel;
//         per_head = 1: one decay a head)
// mode 1: out <- exp(-exp(x + bias[c]))
// x has rows of stride ld, out is contiguous [T, n] (and may be x itself). `steps`
// (mode 0, optional, contiguous [T, n]) receives softplus(x + bias[c]) itself.
__global__ void decay_gate_kernel(const float* in, long long ld, float* out, long long n_total,
                                  int n, int per_head, const float* __restrict__ A,
                                  const float* __restrict__ bias, int mode, float* steps) {
  fb_pdl_launch();
  fb_pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / n;
    const int c = (int)(i - t * n);
    const float v = __ldcg(in + t * ld + c) + bias[c];
    if (mode == 0) {
      const float sp = softplusf_(v);
      out[i] = expf(-expf(A[c / per_head]) * sp);
      if (steps != nullptr) steps[i] = sp;
    } else {
      out[i] = expf(-expf(v));
    }
  }
}

// ------------------------------------------------------------ the recurrences
constexpr int R = 16;  // state rows a thread holds

struct ScanArgs {
  const float* q; long long q_ld;   // [T, *]: query (delta) or receptance (wkv); head h at (h / rep) * dim
  const float* k; long long k_ld;   // keys, same head mapping
  const float* v; long long v_ld;   // values: head h at h * vdim
  const float* g; long long g_ld;   // decays: head h at h * dim, or one per head at h (g_scalar)
  const float* beta; long long beta_ld;  // delta: raw step size per head (sigmoid applied here);
                                    // ssd: the step size per head as it is
  const float* bonus;               // wkv: [H, dim]; ssd: the skip, [H]
  float* state; long long state_stride; long long s_offset;
  float* out;                       // [T, H * vdim]
  const int* cu_tokens; const int* slots;
  int H, rep, dim, vdim;
  int g_scalar;                     // one decay a head instead of one a key channel
};

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_one() {
  asm volatile("cp.async.wait_group 1;" ::: "memory");
}

// The inputs of `tc` tokens at a time are brought into shared memory by
// asynchronous copies (two buffers: the next tokens arrive while these are
// worked), so the token-by-token loop waits for shared memory, not for L2.
// Per token: q [dimp] | k [dimp] | g [dimp] | v [the block's columns] | beta | padding,
// dimp = KP * rp the key rows padded so that lane group `part` holds the rp
// consecutive rows part * rp .. (a multiple of 4: they are read as float4).
// RP: key rows a lane holds (4 or 8, or 16 for heads of more than 256 key channels);
// MINE: elements of a token's record a thread copies at most.
template <int MODE, int KP, int RP, int MINE>
__global__ void __launch_bounds__(256) scan_kernel(ScanArgs a, int tc) {
  constexpr int rp = RP;
  fb_pdl_wait();
  constexpr int COLS_W = 32 / KP;  // columns a warp holds
  extern __shared__ __align__(16) float sbuf[];
  const int seq = blockIdx.x, h = blockIdx.y;
  const int start = a.cu_tokens[seq], n = a.cu_tokens[seq + 1] - start;
  if (n <= 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int part = lane / COLS_W;
  const int cols_blk = nwarps * COLS_W;
  const int col0 = blockIdx.z * cols_blk;
  const int jl = warp * COLS_W + lane % COLS_W;  // column within the block
  const int j = col0 + jl;
  const bool col = j < a.vdim;
  const int dim = a.dim, vdim = a.vdim;
  const int dimp = KP * rp;
  float* S = a.state + (long long)a.slots[seq] * a.state_stride + a.s_offset +
             (long long)h * dim * vdim;
  const long long qoff = (long long)(h / a.rep) * dim, goff = (long long)h * dim;
  const int per_tok = (3 * dimp + cols_blk + 1 + 3) / 4 * 4;
  const int row0 = part * rp;  // this thread's first key row
  // A token's output is a sum over the KP lanes of a column. It is not needed for the
  // next token, so the lanes' shares wait in shared memory and are added up once per
  // chunk of tokens (every lane group takes its share of the chunk's tokens), instead
  // of a chain of shuffles inside every token's step.
  float* opart = sbuf + (size_t)2 * tc * per_tok + (size_t)warp * 32 * tc;  // [tc][32] a warp

  // what a thread copies is the same for every token: its elements of a token's record
  // are found once (at most four a thread), then only the token's row offset changes
  const float* src0[MINE];  // where the thread's element e of the NEXT token to copy lies
  long long ld[MINE];
  int at[MINE];
#pragma unroll
  for (int e = 0; e < MINE; ++e) {
    const int c = threadIdx.x + e * blockDim.x;
    const float* src = nullptr;
    long long step = 0;
    if (c < 3 * dimp) {
      const int which = c / dimp, row = c - which * dimp;
      if (row < dim) {
        src = which == 0 ? a.q + qoff + row : which == 1 ? a.k + qoff + row
                         : a.g_scalar ? a.g + h : a.g + goff + row;
        step = which == 0 ? a.q_ld : which == 1 ? a.k_ld : a.g_ld;
      }
    } else if (c < 3 * dimp + cols_blk) {
      if (col0 + (c - 3 * dimp) < vdim) {
        src = a.v + (size_t)h * vdim + col0 + (c - 3 * dimp);
        step = a.v_ld;
      }
    } else if (MODE != 1 && c == 3 * dimp + cols_blk) {
      src = a.beta + h;
      step = a.beta_ld;
    }
    src0[e] = src == nullptr ? nullptr : src + (size_t)start * step;
    ld[e] = step; at[e] = c < per_tok ? c : -1;
  }
  // (tokens are staged in order, so the source pointers only ever move on by one row)
  auto stage = [&](int buf, int nt) {
    float* dst = sbuf + (size_t)buf * tc * per_tok;
    for (int r = 0; r < nt; ++r, dst += per_tok) {
#pragma unroll
      for (int e = 0; e < MINE; ++e) {
        if (at[e] >= 0) {
          if (src0[e] != nullptr) {
            cp_async4(dst + at[e], src0[e]);
            src0[e] += ld[e];
          } else {
            dst[at[e]] = 0.f;
          }
        }
      }
    }
  };

  const float skip = MODE == 2 ? a.bonus[h] : 0.f;
  float s[RP], bonus[RP];
#pragma unroll
  for (int i = 0; i < RP; ++i) {
    const int row = row0 + i;
    const bool ok = row < dim;
    s[i] = (col && ok) ? S[(size_t)row * vdim + j] : 0.f;
    bonus[i] = (MODE == 1 && ok) ? a.bonus[goff + row] : 0.f;
  }
  stage(0, min(tc, n));
  cp_async_commit();
  for (int c0 = 0; c0 < n; c0 += tc) {
    const int buf = (c0 / tc) & 1, nt = min(tc, n - c0);
    if (c0 + tc < n) stage(buf ^ 1, min(tc, n - c0 - tc));
    cp_async_commit();  // (an empty group when nothing follows: the count below stays right)
    cp_async_wait_but_one();
    __syncthreads();
    const float* tok = sbuf + (size_t)buf * tc * per_tok;
    for (int r = 0; r < nt; ++r, tok += per_tok) {
      const float v = tok[3 * dimp + jl];
      const float4* q4 = reinterpret_cast<const float4*>(tok + row0);
      const float4* k4 = reinterpret_cast<const float4*>(tok + dimp + row0);
      const float4* g4 = reinterpret_cast<const float4*>(tok + 2 * dimp + row0);
      float o4[4] = {0.f, 0.f, 0.f, 0.f};  // four sums side by side: short dependent chains
      if (MODE == 0) {
        float kv4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          {
            const float4 g = g4[i / 4], k = k4[i / 4];
            s[i] *= g.x; s[i + 1] *= g.y; s[i + 2] *= g.z; s[i + 3] *= g.w;
            kv4[0] = fmaf(s[i], k.x, kv4[0]); kv4[1] = fmaf(s[i + 1], k.y, kv4[1]);
            kv4[2] = fmaf(s[i + 2], k.z, kv4[2]); kv4[3] = fmaf(s[i + 3], k.w, kv4[3]);
          }
        }
        float kv = (kv4[0] + kv4[1]) + (kv4[2] + kv4[3]);
#pragma unroll
        for (int off = COLS_W; off < 32; off <<= 1) kv += __shfl_xor_sync(0xffffffffu, kv, off);
        const float u = sigmoidf_(tok[3 * dimp + cols_blk]) * (v - kv);
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          {
            const float4 k = k4[i / 4], q = q4[i / 4];
            s[i] = fmaf(k.x, u, s[i]); s[i + 1] = fmaf(k.y, u, s[i + 1]);
            s[i + 2] = fmaf(k.z, u, s[i + 2]); s[i + 3] = fmaf(k.w, u, s[i + 3]);
            o4[0] = fmaf(s[i], q.x, o4[0]); o4[1] = fmaf(s[i + 1], q.y, o4[1]);
            o4[2] = fmaf(s[i + 2], q.z, o4[2]); o4[3] = fmaf(s[i + 3], q.w, o4[3]);
          }
        }
      } else if (MODE == 2) {
        const float u = tok[3 * dimp + cols_blk] * v;  // step size times the value
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          {
            const float4 g = g4[i / 4], k = k4[i / 4], q = q4[i / 4];
            s[i] = fmaf(k.x, u, g.x * s[i]); s[i + 1] = fmaf(k.y, u, g.y * s[i + 1]);
            s[i + 2] = fmaf(k.z, u, g.z * s[i + 2]); s[i + 3] = fmaf(k.w, u, g.w * s[i + 3]);
            o4[0] = fmaf(s[i], q.x, o4[0]); o4[1] = fmaf(s[i + 1], q.y, o4[1]);
            o4[2] = fmaf(s[i + 2], q.z, o4[2]); o4[3] = fmaf(s[i + 3], q.w, o4[3]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          {
            const float4 g = g4[i / 4], k = k4[i / 4], q = q4[i / 4];
            const float kv0 = k.x * v, kv1 = k.y * v, kv2 = k.z * v, kv3 = k.w * v;
            o4[0] = fmaf(q.x, fmaf(bonus[i], kv0, s[i]), o4[0]);
            o4[1] = fmaf(q.y, fmaf(bonus[i + 1], kv1, s[i + 1]), o4[1]);
            o4[2] = fmaf(q.z, fmaf(bonus[i + 2], kv2, s[i + 2]), o4[2]);
            o4[3] = fmaf(q.w, fmaf(bonus[i + 3], kv3, s[i + 3]), o4[3]);
            s[i] = fmaf(g.x, s[i], kv0); s[i + 1] = fmaf(g.y, s[i + 1], kv1);
            s[i + 2] = fmaf(g.z, s[i + 2], kv2); s[i + 3] = fmaf(g.w, s[i + 3], kv3);
          }
        }
      }
      opart[r * 32 + lane] = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    }
    __syncwarp();
    for (int r = part; r < nt; r += KP) {
      float o = 0.f;
#pragma unroll
      for (int p = 0; p < KP; ++p) o += opart[r * 32 + p * COLS_W + (lane % COLS_W)];
      if (MODE == 2)  // the skip: the token's own value straight to its output
        o = fmaf(skip, sbuf[(size_t)buf * tc * per_tok + (size_t)r * per_tok + 3 * dimp + jl], o);
      if (col) a.out[(size_t)(start + c0 + r) * a.H * vdim + (size_t)h * vdim + j] = o;
    }
    __syncthreads();  // the buffers are refilled by the next iteration
  }
#pragma unroll
  for (int i = 0; i < RP; ++i) {
    const int row = row0 + i;
    if (col && row < dim) S[(size_t)row * vdim + j] = s[i];
  }
}

// ------------------------------------------------- per-head RMS norm and gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w[h * w_stride + :] * act(gate[t, h, :])
// act: 0 sigmoid, 1 SiLU. `gate_first`: the gate comes before the norm,
// out = y / sqrt(mean(y^2) + eps) * w with y = o * act(gate). A "head" is any equal part
// of the row that is normalised by itself. Output rows lie `out_ld` elements apart and
// are multiplied by `out_scale` before they are rounded.
// HG_HOLD: elements of a head a lane holds (heads of up to 32 * HG_HOLD; 0: any size, the
// head is read twice)
template <typename T, int HG_HOLD>
__global__ void head_norm_gate_kernel(const float* o, const float* __restrict__ w, int w_stride,
                                      const float* gate, long long gate_ld, int act, float eps,
                                      T* __restrict__ out, long long out_ld, float out_scale,
                                      int H, int vdim, int gate_first) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  // a warp a head; the heads of a token are spread over blockIdx.y
  for (int h = blockIdx.y * nwarps + warp; h < H; h += gridDim.y * nwarps) {
    const float* row = o + ((size_t)t * H + h) * vdim;
    if constexpr (HG_HOLD > 0) {
      // a lane holds its elements: every load of the head is on its way before the first
      // is used, and nothing is read twice
      float v[HG_HOLD], ga[HG_HOLD], wv[HG_HOLD];
#pragma unroll
      for (int i = 0; i < HG_HOLD; ++i) {
        const int d = lane + 32 * i;
        const bool in = d < vdim;
        v[i] = in ? __ldcg(row + d) : 0.f;
        ga[i] = in ? __ldcg(gate + (size_t)t * gate_ld + (size_t)h * vdim + d) : 0.f;
        wv[i] = in ? w[(size_t)h * w_stride + d] : 0.f;
      }
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < HG_HOLD; ++i) {
        ga[i] = act == 0 ? sigmoidf_(ga[i]) : ga[i] * sigmoidf_(ga[i]);
        if (gate_first) v[i] *= ga[i];
        ss += v[i] * v[i];
      }
      const float r = 1.0f / sqrtf(fb_warp_sum(ss) / (float)vdim + eps);
#pragma unroll
      for (int i = 0; i < HG_HOLD; ++i) {
        const int d = lane + 32 * i;
        // (gate first: v already carries the gate)
        if (d < vdim)
          out[(size_t)t * out_ld + (size_t)h * vdim + d] =
              fb_from_float<T>(v[i] * r * wv[i] * (gate_first ? 1.0f : ga[i]) * out_scale);
      }
    } else {
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) {
      float v = __ldcg(row + d);
      if (gate_first) {
        const float gz = __ldcg(gate + (size_t)t * gate_ld + (size_t)h * vdim + d);
        v *= act == 0 ? sigmoidf_(gz) : gz * sigmoidf_(gz);
      }
      ss += v * v;
    }
    const float r = 1.0f / sqrtf(fb_warp_sum(ss) / (float)vdim + eps);
    for (int d = lane; d < vdim; d += 32) {
      const float gz = __ldcg(gate + (size_t)t * gate_ld + (size_t)h * vdim + d);
      const float ga = act == 0 ? sigmoidf_(gz) : gz * sigmoidf_(gz);
      out[(size_t)t * out_ld + (size_t)h * vdim + d] =
          fb_from_float<T>(__ldcg(row + d) * r * w[(size_t)h * w_stride + d] * ga * out_scale);
    }
    }
  }
}

// out = act(in) rounded to the activation type; act: 0 identity, 1 tanh, 2 the square of relu
template <typename T>
__global__ void unary_cast_kernel(const float* in, long long ld, T* __restrict__ out, int n,
                                  int act) {
  fb_pdl_launch();
  fb_pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
    const float v = __ldcg(in + t * ld + i);
    const float r = fmaxf(v, 0.f);
    out[t * n + i] = fb_from_float<T>(act == 1 ? tanhf(v) : act == 2 ? r * r : v);
  }
}

// x[t, i] <- x[t, i] * sigmoid(gate[t, i]), in place: x in the activation type, the gate's
// rows float32; the product is made in 32-bit and rounded once.
template <typename T>
__global__ void sigmoid_gate_kernel(T* x, long long ldx, const float* gate, long long ldg, int n) {
  fb_pdl_launch();
  fb_pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
    const float g = __ldcg(gate + t * ldg + i);
    const float v = fb_to_float<T>(x[t * ldx + i]);
    x[t * ldx + i] = fb_from_float<T>(v / (1.0f + expf(-g)));
  }
}
}  // namespace

FB_API int fb_sigmoid_gate(void* x, int dtype, long long ldx, const float* gate, long long ldg,
                           int T, int n, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && n > 0 && ldx >= n && ldg >= n, "sigmoid_gate: bad sizes");
  if (T == 0) return 0;
  const int want = (n + 511) / 512;
  const int parts = T >= 1024 ? (want < 4 ? want : 4) : (want < 64 ? want : 64);
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(sigmoid_gate_kernel<E>, dim3(T, parts), dim3(256), 0, stream,
      (E*)x, ldx, gate, ldg, n)));
  return fb_check_launch("sigmoid_gate");
}

FB_API int fb_token_shift_mix(const void* h, int dtype, float* state, long long state_stride,
                              long long prev_offset, const float* mu, void* out,
                              const int* seq_of_token, const int* cu_tokens, const int* slots,
                              int T, int W, int n_mix, int single, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0 && n_mix > 0, "token_shift_mix: bad sizes");
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(token_shift_mix_kernel<E>, dim3(T), dim3(256), 0, stream,
      (const E*)h, state, state_stride, prev_offset, mu, (E*)out, seq_of_token, cu_tokens, slots,
      T, W, n_mix, single)));
  return fb_check_launch("token_shift_mix");
}

FB_API int fb_state_tail_update(const void* x, int dtype, long long ld, float* state,
                                long long state_stride, long long offset, int n_tail, int C,
                                const int* cu_tokens, const int* slots, int n_seqs,
                                cudaStream_t stream) {
  FB_REQUIRE(n_seqs >= 0 && C > 0 && n_tail >= 0 && ld >= C, "state_tail_update: bad sizes");
  if (n_seqs == 0 || n_tail == 0) return 0;
  dim3 grid(n_seqs, (C + 255) / 256 < 64 ? (C + 255) / 256 : 64);
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(state_tail_update_kernel<E>, dim3(grid), dim3(256), 0,
      stream, (const E*)x, ld, state, state_stride, offset, n_tail, C, cu_tokens, slots)));
  return fb_check_launch("state_tail_update");
}

FB_API int fb_conv_silu_unit(const float* x, long long ld, const float* w, const float* bias, int taps,
                             float* state, long long state_stride, long long tail_offset,
                             float* out, int C, const int* seq_of_token, const int* cu_tokens,
                             const int* slots, int n_unit, int dim, int n_scaled, float extra,
                             float unit_eps, int T, int single, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && C > 0 && taps >= 1 && ld >= C, "conv_silu_unit: bad sizes");
  FB_REQUIRE(n_unit >= 0 && (long long)n_unit * dim <= C && n_scaled <= n_unit,
             "conv_silu_unit: %d unit heads of %d exceed %d channels", n_unit, dim, C);
  FB_REQUIRE(n_unit == 0 || (size_t)C * 4 <= 200 * 1024,
             "conv_silu_unit: %d channels do not fit shared memory", C);
  if (T == 0) return 0;
  if (n_unit == 0) {
    fb_launch(conv_silu_kernel, dim3(T, (C + 255) / 256), dim3(256), 0, stream, x, ld, w, bias, taps,
              state, state_stride, tail_offset, out, C, seq_of_token, cu_tokens, slots, single);
    return fb_check_launch("conv_silu");
  }
  const size_t smem = (size_t)C * 4;
  static bool seen[64];
  if (smem > 48 * 1024 && fb_first_use_on_device(seen))
    cudaFuncSetAttribute(conv_silu_unit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
  // few tokens: wide blocks, so that a token's loads are many threads' and not one
  // thread's one after another
  const int threads = (T <= 64 && C >= 2048) ? 1024 : 256;
  fb_launch(conv_silu_unit_kernel, dim3(T), dim3(threads), smem, stream, x, ld, w, bias, taps, state,
            state_stride, tail_offset, out, C, seq_of_token, cu_tokens, slots, n_unit, dim,
            n_scaled, extra, unit_eps, single);
  return fb_check_launch("conv_silu_unit");
}

FB_API int fb_decay_gate(const float* x, long long ld, float* out, int T, int n, int per_head,
                         const float* A, const float* bias, int mode, float* steps,
                         cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && n > 0 && per_head > 0 && bias != nullptr && (mode == 1 || A != nullptr) &&
             ld >= n, "decay_gate: bad arguments");
  if (T == 0) return 0;
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
  fb_launch(decay_gate_kernel, dim3(blocks), dim3(256), 0, stream, x, ld, out, total, n, per_head,
            A, bias, mode, steps);
  return fb_check_launch("decay_gate");
}

namespace {
// A long scan (a prompt) is launched without the dependent-launch mark: placed early
// behind the short kernels in front of it, its few long-running blocks were seen to take
// twice their time (a 2,048-token prompt's scan 0.71 ms alone, 1.6 ms in the step).
template <typename K, typename... Args>
inline void launch_scan(K kernel, bool serial, dim3 grid, dim3 block, size_t smem,
                        cudaStream_t stream, Args&&... args) {
  if (serial) fb_launch_serial(kernel, grid, block, smem, stream, std::forward<Args>(args)...);
  else fb_launch(kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}
}  // namespace

FB_API int fb_state_scan(int mode, const float* q, long long q_ld, const float* k, long long k_ld,
                         const float* v, long long v_ld, const float* g, long long g_ld,
                         const float* beta, long long beta_ld, const float* bonus, float* state,
                         long long state_stride, long long s_offset, float* out,
                         const int* cu_tokens, const int* slots, int n_seqs, int H, int rep,
                         int dim, int vdim, int g_scalar, int serial_launch, cudaStream_t stream) {
  const bool serial = serial_launch != 0;
  FB_REQUIRE(mode >= 0 && mode <= 2, "state_scan: unknown recurrence %d", mode);
  FB_REQUIRE(mode != 2 || g_scalar, "state_scan: the state-space recurrence takes one decay a head");
  FB_REQUIRE(n_seqs >= 0 && H > 0 && rep > 0 && H % rep == 0 && dim > 0 && vdim > 0,
             "state_scan: bad sizes");
  FB_REQUIRE(dim <= R * 32, "state_scan: %d key channels exceed %d", dim, R * 32);
  FB_REQUIRE((mode == 1 || beta != nullptr) && (mode == 0 || bonus != nullptr),
             "state_scan: a missing input");
  if (n_seqs == 0) return 0;
  ScanArgs a{q, q_ld, k, k_ld, v, v_ld, g, g_ld, beta, beta_ld, bonus, state, state_stride,
             s_offset, out, cu_tokens, slots, H, rep, dim, vdim, g_scalar ? 1 : 0};
  // a column is shared by kp lanes: eight key rows a lane where the head allows it
  // (a token's step is a chain of dependent instructions; fewer rows a lane shorten it)
  int kp = 1;
  while (kp * 8 < dim && kp < 32) kp *= 2;
  // few blocks (a prompt of one or two sequences): four rows a lane make twice the
  // warps with half the work each, which is what fills an SM's schedulers then
  {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess)
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int cols_blk8 = 4 * (32 / kp);
    const long long blocks = (long long)n_seqs * H * ((vdim + cols_blk8 - 1) / cols_blk8);
    if (blocks < 2LL * sms && kp < 32 && (dim + 2 * kp - 1) / (2 * kp) <= 4) kp *= 2;
  }
  const int cols_w = 32 / kp;
  const int warps_needed = (vdim + cols_w - 1) / cols_w;
  const int most = kp >= 16 ? 8 : 4;  // (a wide head's record takes more threads to copy)
  const int warps = warps_needed < most ? warps_needed : most;
  dim3 grid(n_seqs, H, (warps_needed + warps - 1) / warps);
  // key rows a lane holds: 4 or 8, or 16 for heads of more than 256 key channels
  const int rows = (dim + kp - 1) / kp;
  const int rp = rows <= 4 ? 4 : rows <= 8 ? 8 : 16;
  // tokens staged at a time: two buffers within the 48 KB that need no opt-in
  const int per_tok = (3 * kp * rp + warps * cols_w + 1 + 3) / 4 * 4;
  int tc = 16;
  while (tc > 1 && (size_t)2 * tc * per_tok * 4 > 48 * 1024) tc /= 2;
  while (tc > 1 && (size_t)(2 * tc * per_tok + warps * 32 * tc) * 4 > 48 * 1024) tc /= 2;
  const size_t smem = (size_t)(2 * tc * per_tok + warps * 32 * tc) * 4;
  FB_REQUIRE(smem <= 48 * 1024, "state_scan: a token's inputs (%d floats) do not fit", per_tok);
  const int mine = (per_tok + warps * 32 - 1) / (warps * 32);
  FB_REQUIRE(mine <= 8, "state_scan: %d inputs a token are more than the block's threads copy",
             per_tok);
#define FB_SCAN_LAUNCH(M_, KP_, RP_, MINE_) \
  launch_scan(scan_kernel<M_, KP_, RP_, MINE_>, serial, grid, dim3(warps * 32), smem, stream, a, tc)
#define FB_SCAN_MINE(M_, KP_, RP_)                       \
  do {                                                   \
    if (mine <= 2) FB_SCAN_LAUNCH(M_, KP_, RP_, 2);      \
    else FB_SCAN_LAUNCH(M_, KP_, RP_, 8);                \
  } while (0)
#define FB_SCAN(KP_)                                                \
  case KP_:                                                         \
    if (rp == 4) { if (mode == 0) FB_SCAN_MINE(0, KP_, 4); else if (mode == 1) FB_SCAN_MINE(1, KP_, 4); else FB_SCAN_MINE(2, KP_, 4); } \
    else { if (mode == 0) FB_SCAN_MINE(0, KP_, 8); else if (mode == 1) FB_SCAN_MINE(1, KP_, 8); else FB_SCAN_MINE(2, KP_, 8); }         \
    break;
  if (kp == 32 && rp == 16) {
    if (mode == 0) FB_SCAN_MINE(0, 32, 16); else if (mode == 1) FB_SCAN_MINE(1, 32, 16); else FB_SCAN_MINE(2, 32, 16);
  } else {
    switch (kp) {
      FB_SCAN(1) FB_SCAN(2) FB_SCAN(4) FB_SCAN(8) FB_SCAN(16) FB_SCAN(32)
      default: return fb_fail(1, "state_scan: no kernel for %d lanes a column", kp);
    }
  }
#undef FB_SCAN
#undef FB_SCAN_MINE
#undef FB_SCAN_LAUNCH
  return fb_check_launch("state_scan");
}

FB_API int fb_head_norm_gate(const float* o, const float* w, int w_stride, const float* gate,
                             long long gate_ld, int act, float eps, void* out, long long out_ld,
                             float out_scale, int dtype, int T, int H, int vdim, int gate_first,
                             cudaStream_t stream) {
  FB_REQUIRE(out_ld >= (long long)H * vdim, "head_norm_gate: output rows of %lld are too short", out_ld);
  FB_REQUIRE(T >= 0 && H > 0 && vdim > 0 && (act == 0 || act == 1), "head_norm_gate: bad sizes");
  if (T == 0) return 0;
  // few tokens: a token's heads go to several blocks, so that their loads run side by side
  const int parts = T <= 256 ? (H + 7) / 8 : 1;
#define FB_HEAD_NORM_GATE(E, HOLD)                                                             \
  fb_launch(head_norm_gate_kernel<E, HOLD>, dim3(T, parts), dim3(256), 0, stream, o, w, w_stride, \
            gate, gate_ld, act, eps, (E*)out, out_ld, out_scale, H, vdim, gate_first)
  FB_DISPATCH_DTYPE(dtype, E, {
    if (vdim <= 64) FB_HEAD_NORM_GATE(E, 2);
    else if (vdim <= 128) FB_HEAD_NORM_GATE(E, 4);
    else if (vdim <= 256) FB_HEAD_NORM_GATE(E, 8);
    else if (vdim <= 512) FB_HEAD_NORM_GATE(E, 16);
    else FB_HEAD_NORM_GATE(E, 0);
  });
#undef FB_HEAD_NORM_GATE
  return fb_check_launch("head_norm_gate");
}

FB_API int fb_unary_cast(const float* in, long long ld, void* out, int dtype, int T, int n, int act,
                         cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && n > 0 && ld >= n, "unary_cast: bad sizes");
  if (T == 0) return 0;
  const int want = (n + 511) / 512;  // two elements a thread, unless the rows alone fill the device
  const int parts = T >= 1024 ? (want < 4 ? want : 4) : (want < 64 ? want : 64);
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(unary_cast_kernel<E>, dim3(T, parts), dim3(256), 0, stream, in,
      ld, (E*)out, n, act)));
  return fb_check_launch("unary_cast");
}
