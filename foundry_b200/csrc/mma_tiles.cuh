// Pieces of the mma.sync attention kernels that several files share: asynchronous
// 16-byte copies into shared memory, ldmatrix, the bf16 m16n8k16 product with 32-bit
// sums, and swizzled [rows, P] bfloat16 tiles whose pitch P is the row's size rounded
// up to a power of two.
#pragma once
#include "common.cuh"

namespace fb_mma {

constexpr int THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__host__ __device__ constexpr int pitch_of(int d) { return d <= 16 ? 16 : d <= 32 ? 32 : d <= 64 ? 64 : d <= 128 ? 128 : 256; }

// Shared-memory layout of a [rows, P] bfloat16 tile (P a power of two, the row's
// elements padded up to it): 16-byte chunks of a row are XORed with low bits of the row.
template <int P>
struct Swz {
  static constexpr int CHUNKS = P / 8;
  static constexpr int MASK = CHUNKS >= 8 ? 7 : CHUNKS - 1;
  static constexpr int SHIFT = CHUNKS >= 8 ? 0 : (CHUNKS == 4 ? 1 : 2);
  __device__ static __forceinline__ int off(int row, int col) {
    const int chunk = col >> 3;
    return row * P + (((chunk ^ ((row >> SHIFT) & MASK))) << 3) + (col & 7);
  }
};

// Copies columns [0, cols) of `rows` rows (row stride `ld`) into columns [col0, col0 + cols)
// of a swizzled tile; rows at or beyond `valid_rows` are zero-filled. cols is a multiple of 8.
template <int P>
__device__ __forceinline__ void load_cols(__nv_bfloat16* dst, const __nv_bfloat16* src,
                                          long long ld, int rows, int valid_rows, int cols,
                                          int col0) {
  const int ch = cols / 8;
  for (int id = threadIdx.x; id < rows * ch; id += THREADS) {
    const int r = id / ch, c = id - r * ch;
    const bool ok = r < valid_rows;
    const __nv_bfloat16* s = src + (ok ? (long long)r * ld + c * 8 : 0);
    cp_async16(smem_u32(dst + Swz<P>::off(r, col0 + c * 8)), s, ok);
  }
}

}  // namespace fb_mma
