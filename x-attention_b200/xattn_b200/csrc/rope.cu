// Rotary position embedding applied IN PLACE to the query and key projections, one launch for both.
//
// Replaces apply_rotary_pos_emb of the reference's Llama patch (xattn/src/load_llama.py:34-65, call site :142):
//     x' = x * cos + rotate_half(x) * sin,   rotate_half(x) = cat(-x[D/2:], x[:D/2])
// evaluated there as three 16-bit torch operations, each of which rounds its fp32 result to the storage type.
// The kernel keeps exactly those roundings, so its output equals the reference's bit for bit:
//     x'[i]       = rn(rn(x[i]       * cos[i])       + rn(-x[i + D/2] * sin[i]))          i <  D/2
//     x'[i + D/2] = rn(rn(x[i + D/2] * cos[i + D/2]) + rn( x[i]       * sin[i + D/2]))
// The projections leave q and k as [B, L, H*D] rows; the attention kernels read any [B, H, L, D] view with unit
// stride on D through their tensor maps, so the rotated tensors need no transposed copy afterwards.
//
// HBM-bound: every element of q and k is read once and written once (cos/sin rows are shared by the heads of a
// token and stay in L2).  A thread owns 8 elements of the first half of a row and the 8 partners in the second
// half (two 16-byte loads, two 16-byte stores).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.cuh"

namespace xb {

struct RopeParams {
  void* x[2];                 // q, k
  int heads[2];
  int64_t sb[2], sh[2], sl[2];
  const void* cos;
  const void* sin;
  int64_t cs_b, cs_l;         // element strides of cos/sin [B, L, D]
  int batch, len, head_dim;
  long long work[2];          // 16-byte vector pairs of q, of q and k together
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) rope_qk_kernel(const RopeParams p) {
  const int vec_per_row = p.head_dim / 16;          // vector pairs per (token, head) row
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < p.work[1];
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int which = e >= p.work[0] ? 1 : 0;
    long long r = which ? e - p.work[0] : e;
    const int v = static_cast<int>(r % vec_per_row);
    r /= vec_per_row;
    const int h = static_cast<int>(r % p.heads[which]);
    r /= p.heads[which];
    const int l = static_cast<int>(r % p.len);
    const int b = static_cast<int>(r / p.len);
    T* row = static_cast<T*>(p.x[which]) + b * p.sb[which] + h * p.sh[which] + l * p.sl[which];
    const T* c = static_cast<const T*>(p.cos) + b * p.cs_b + l * p.cs_l;
    const T* s = static_cast<const T*>(p.sin) + b * p.cs_b + l * p.cs_l;
    const int half = p.head_dim / 2;
    const int i0 = v * 8;
    union V16 { uint4 u; T t[8]; };
    V16 x1, x2, c1, c2, s1, s2, o1, o2;
    x1.u = *reinterpret_cast<const uint4*>(row + i0);
    x2.u = *reinterpret_cast<const uint4*>(row + half + i0);
    c1.u = __ldg(reinterpret_cast<const uint4*>(c + i0));
    c2.u = __ldg(reinterpret_cast<const uint4*>(c + half + i0));
    s1.u = __ldg(reinterpret_cast<const uint4*>(s + i0));
    s2.u = __ldg(reinterpret_cast<const uint4*>(s + half + i0));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = to_f32(x1.t[i]), d = to_f32(x2.t[i]);
      // every product and the sum are rounded to the storage type, as the reference's 16-bit tensor ops do
      const float p1 = to_f32(from_f32<T>(a * to_f32(c1.t[i])));
      const float r1 = to_f32(from_f32<T>(-d * to_f32(s1.t[i])));
      const float p2 = to_f32(from_f32<T>(d * to_f32(c2.t[i])));
      const float r2 = to_f32(from_f32<T>(a * to_f32(s2.t[i])));
      o1.t[i] = from_f32<T>(p1 + r1);
      o2.t[i] = from_f32<T>(p2 + r2);
    }
    *reinterpret_cast<uint4*>(row + i0) = o1.u;
    *reinterpret_cast<uint4*>(row + half + i0) = o2.u;
  }
}

int rope_qk_launch(void* q, void* k, int dtype, int batch, int hq, int hkv, int len, int head_dim, int64_t qsb,
                   int64_t qsh, int64_t qsl, int64_t ksb, int64_t ksh, int64_t ksl, const void* cos, const void* sin,
                   int64_t cs_stride_b, int64_t cs_stride_l, cudaStream_t stream) {
  if (!q || !k || !cos || !sin) return XATTN_B200_ERR_ARG;
  if (dtype != XATTN_B200_BF16 && dtype != XATTN_B200_F16) return XATTN_B200_ERR_ARG;
  if (batch < 1 || hq < 1 || hkv < 1 || len < 1 || head_dim < 16 || head_dim % 16 != 0) return XATTN_B200_ERR_ARG;
  // 16-byte vectors: aligned bases, strides that are multiples of 8 elements
  const uintptr_t bases = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(cos) | reinterpret_cast<uintptr_t>(sin);
  if (bases & 15) return XATTN_B200_ERR_ARG;
  if ((qsb | qsh | qsl | ksb | ksh | ksl | cs_stride_b | cs_stride_l) & 7) return XATTN_B200_ERR_ARG;
  RopeParams p;
  p.x[0] = q; p.x[1] = k;
  p.heads[0] = hq; p.heads[1] = hkv;
  p.sb[0] = qsb; p.sh[0] = qsh; p.sl[0] = qsl;
  p.sb[1] = ksb; p.sh[1] = ksh; p.sl[1] = ksl;
  p.cos = cos; p.sin = sin; p.cs_b = cs_stride_b; p.cs_l = cs_stride_l;
  p.batch = batch; p.len = len; p.head_dim = head_dim;
  const long long per_head = static_cast<long long>(batch) * len * (head_dim / 16);
  p.work[0] = per_head * hq;
  p.work[1] = per_head * (hq + hkv);
  const int block = 256;
  long long blocks = (p.work[1] + block - 1) / block;
  const long long cap = static_cast<long long>(sm_count()) * 16;      // grid-stride beyond 16 CTAs per SM
  if (blocks > cap) blocks = cap;
  if (dtype == XATTN_B200_BF16)
    rope_qk_kernel<__nv_bfloat16><<<static_cast<int>(blocks), block, 0, stream>>>(p);
  else
    rope_qk_kernel<__half><<<static_cast<int>(blocks), block, 0, stream>>>(p);
  return launch_status();
}

}  // namespace xb
