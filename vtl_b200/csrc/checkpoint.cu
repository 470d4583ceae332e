// Checkpoint tensor payloads on the device.  The reference stores every tensor as text:
// each element widened to f64, its 8 bytes most significant first, the byte string in
// standard base64 with '=' padding (encode_tensor / decode_tensor,
// nn/models/serialization.v:421-473).  Encoding and decoding 134 M parameters this way is
// 0.5 GB in and 1.4 GB out of pure byte shuffling, bound by HBM: it runs here, next to the
// parameters, and only the text crosses PCIe.
//
// Work split: 3 elements = 24 bytes = 32 base64 characters per thread, so every thread writes
// (reads, when decoding) two aligned 16-byte pieces of text and no base64 group straddles two
// threads.  Only the last thread sees a short group and the padding.
#include "common.cuh"

namespace {

__host__ __device__ inline size_t b64_len(size_t n) { return (n * 8 + 2) / 3 * 4; }

// Four 6-bit values, one per byte -> their four characters of the standard alphabet, all bytes at
// once.  (v + 128 - k) has bit 7 set exactly when v >= k, so the range tests cost one add each;
// 'A'+v for v < 26, 'a'+v-26 (= v+71) below 52, '0'+v-52 (= v-4) below 62, then '+' and '/'.
// No byte ever carries or borrows: v + 65 + 6 <= 134, and what is subtracted never exceeds it.
__device__ __forceinline__ uint32_t b64_chars4(uint32_t v4) {
  const uint32_t ge26 = ((v4 + 0x66666666u) >> 7) & 0x01010101u;
  const uint32_t ge52 = ((v4 + 0x4c4c4c4cu) >> 7) & 0x01010101u;
  const uint32_t ge62 = ((v4 + 0x42424242u) >> 7) & 0x01010101u;
  const uint32_t ge63 = ((v4 + 0x41414141u) >> 7) & 0x01010101u;
  return (v4 + 0x41414141u + ge26 * 6u) - (ge52 * 75u + ge62 * 15u - ge63 * 3u);
}
// Four characters, one per byte -> their four 6-bit values, all bytes at once; *bad becomes
// non-zero when a byte is outside the alphabet.  Same carry trick as above on bytes below 128
// (bytes with the top bit set are invalid anyway and are masked out first).
__device__ __forceinline__ uint32_t b64_vals4(uint32_t c4, uint32_t* bad) {
  const uint32_t hi = c4 & 0x80808080u;
  const uint32_t c = c4 & 0x7f7f7f7fu;
#define VTLB_GE(k) (((c + (uint32_t)(128 - (k)) * 0x01010101u) >> 7) & 0x01010101u)
  const uint32_t upper = VTLB_GE('A') & ~VTLB_GE('Z' + 1);
  const uint32_t lower = VTLB_GE('a') & ~VTLB_GE('z' + 1);
  const uint32_t digit = VTLB_GE('0') & ~VTLB_GE('9' + 1);
  const uint32_t plus = VTLB_GE('+') & ~VTLB_GE('+' + 1);
  const uint32_t slash = VTLB_GE('/') & ~VTLB_GE('/' + 1);  // '/' + 1 == '0'
#undef VTLB_GE
  const uint32_t valid = upper | lower | digit | plus | slash;
  *bad |= hi | (valid ^ 0x01010101u);
  // 'A'->0, 'a'->26, '0'->52, '+'->62, '/'->63; per byte the sum added never carries (<= 127 + 19)
  // and what is subtracted never exceeds it for a valid byte (nothing is subtracted otherwise)
  return ((c + digit * 4u + plus * 19u + slash * 16u) - (upper * 65u + lower * 71u)) & 0x3f3f3f3fu;
}

// The 32 characters of three f64 bit patterns (most significant byte first), packed four to a word
// in memory order (first character in the low byte).
__device__ __forceinline__ void encode3(const unsigned long long (&bits)[3], uint32_t (&out)[8]) {
  // the 192 bits as six 32-bit words, big-endian order
  const uint32_t w[6] = {(uint32_t)(bits[0] >> 32), (uint32_t)bits[0], (uint32_t)(bits[1] >> 32),
                         (uint32_t)bits[1],         (uint32_t)(bits[2] >> 32), (uint32_t)bits[2]};
#pragma unroll
  for (int g = 0; g < 8; ++g) {  // characters 4g .. 4g+3 = bits 24g .. 24g+23
    const int bit0 = 24 * g, wi = bit0 >> 5, sh = bit0 & 31;
    // 24 bits starting at bit `sh` of word wi (bit 0 = most significant)
    const unsigned long long two = ((unsigned long long)w[wi] << 32) | (wi + 1 < 6 ? w[wi + 1] : 0u);
    const uint32_t t = (uint32_t)(two >> (40 - sh)) & 0xffffffu;
    out[g] = b64_chars4((t >> 18) | (((t >> 12) & 63u) << 8) | (((t >> 6) & 63u) << 16) | ((t & 63u) << 24));
  }
}

__global__ void __launch_bounds__(256) ckpt_encode_kernel(const float* __restrict__ src, size_t n,
                                                          unsigned char* __restrict__ out) {
  const size_t groups = (n + 2) / 3;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < groups;
       t += (size_t)gridDim.x * blockDim.x) {
    const size_t e0 = t * 3;
    const int have = n - e0 >= 3 ? 3 : (int)(n - e0);
    unsigned long long bits[3] = {0ull, 0ull, 0ull};
#pragma unroll
    for (int j = 0; j < 3; ++j)
      if (j < have) bits[j] = (unsigned long long)__double_as_longlong((double)src[e0 + j]);
    uint32_t ch[8];
    encode3(bits, ch);
    unsigned char* dst = out + t * 32;
    if (have == 3) {
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(ch[0], ch[1], ch[2], ch[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(ch[4], ch[5], ch[6], ch[7]);
    } else {
      // 8 bytes -> 11 characters + "=", 16 bytes -> 22 characters + "=="
      const int nchar = have == 1 ? 11 : 22, total = have == 1 ? 12 : 24;
      for (int i = 0; i < total; ++i)
        dst[i] = i < nchar ? (unsigned char)(ch[i >> 2] >> (8 * (i & 3))) : (unsigned char)'=';
    }
  }
}

// flags: bit 0 = a character outside the alphabet, bit 1 = malformed padding
__global__ void __launch_bounds__(256) ckpt_decode_kernel(const unsigned char* __restrict__ text, size_t n,
                                                          float* __restrict__ dst, uint32_t* __restrict__ flags) {
  const size_t groups = (n + 2) / 3;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < groups;
       t += (size_t)gridDim.x * blockDim.x) {
    const size_t e0 = t * 3;
    const int have = n - e0 >= 3 ? 3 : (int)(n - e0);
    const unsigned char* srcp = text + t * 32;
    uint32_t ch[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int nchar = 32;
    if (have == 3) {
      const uint4 a = reinterpret_cast<const uint4*>(srcp)[0], b = reinterpret_cast<const uint4*>(srcp)[1];
      ch[0] = a.x, ch[1] = a.y, ch[2] = a.z, ch[3] = a.w;
      ch[4] = b.x, ch[5] = b.y, ch[6] = b.z, ch[7] = b.w;
    } else {
      nchar = have == 1 ? 11 : 22;
      const int total = have == 1 ? 12 : 24;
      for (int i = 0; i < total; ++i) {
        const uint32_t c = srcp[i];
        if (i < nchar)
          ch[i >> 2] |= c << (8 * (i & 3));
        else if (c != '=')
          atomicOr(flags, 2u);
      }
    }
    // four characters -> 24 bits; eight such groups -> three 64-bit patterns, most significant first
    uint32_t bad = 0, t24[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      uint32_t c4 = ch[g];
      const int valid_chars = nchar - 4 * g;  // of this group; the rest is padding or absent
      if (valid_chars < 4) {
        const uint32_t keep = valid_chars <= 0 ? 0u : (1u << (8 * valid_chars)) - 1u;
        c4 = (c4 & keep) | (0x41414141u & ~keep);  // 'A' = value 0 where there is no character
      }
      const uint32_t v4 = b64_vals4(c4, &bad);
      t24[g] = ((v4 & 0xffu) << 18) | (((v4 >> 8) & 0xffu) << 12) | (((v4 >> 16) & 0xffu) << 6) | (v4 >> 24);
    }
    unsigned long long bits[3];
    bits[0] = ((unsigned long long)t24[0] << 40) | ((unsigned long long)t24[1] << 16) | (t24[2] >> 8);
    bits[1] = ((unsigned long long)(t24[2] & 0xffu) << 56) | ((unsigned long long)t24[3] << 32) |
              ((unsigned long long)t24[4] << 8) | (t24[5] >> 16);
    bits[2] = ((unsigned long long)(t24[5] & 0xffffu) << 48) | ((unsigned long long)t24[6] << 24) | t24[7];
    if (bad) atomicOr(flags, 1u);
#pragma unroll
    for (int j = 0; j < 3; ++j)
      if (j < have) dst[e0 + j] = (float)__longlong_as_double((long long)bits[j]);  // vtl.cast[T]: plain conversion
  }
}

int ckpt_grid(vtlb_ctx* ctx, size_t groups) {
  size_t b = (groups + 255) / 256;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

}  // namespace

VTLB_API size_t vtlb_ckpt_text_len(size_t n) { return b64_len(n); }

VTLB_API int vtlb_ckpt_encode_f32(vtlb_ctx* ctx, const void* d_src, size_t n, void* d_text) {
  VTLB_ENTER(ctx);
  if (n == 0) return VTLB_OK;
  if (!d_src || !d_text) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_ckpt_encode_f32: null pointer");
  if (!vtlb_aligned16(d_text)) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_ckpt_encode_f32: text buffer not 16-byte aligned");
  ckpt_encode_kernel<<<ckpt_grid(ctx, (n + 2) / 3), 256, 0, ctx->stream>>>((const float*)d_src, n,
                                                                          (unsigned char*)d_text);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_ckpt_decode_f32(vtlb_ctx* ctx, const void* d_text, size_t text_len, void* d_dst, size_t n) {
  VTLB_ENTER(ctx);
  if (text_len != b64_len(n))
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_ckpt_decode_f32: %zu characters cannot hold %zu values (%zu expected)",
                     text_len, n, b64_len(n));
  if (n == 0) return VTLB_OK;
  if (!d_text || !d_dst) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_ckpt_decode_f32: null pointer");
  if (!vtlb_aligned16(d_text)) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_ckpt_decode_f32: text buffer not 16-byte aligned");
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, 256, &scr);
  if (rc) return rc;
  uint32_t* d_flags = (uint32_t*)scr;
  VTLB_CUDA(ctx, cudaMemsetAsync(d_flags, 0, sizeof(uint32_t), ctx->stream));
  ckpt_decode_kernel<<<ckpt_grid(ctx, (n + 2) / 3), 256, 0, ctx->stream>>>((const unsigned char*)d_text, n,
                                                                          (float*)d_dst, d_flags);
  VTLB_LAUNCHED(ctx);
  uint32_t flags = 0;
  VTLB_CUDA(ctx, cudaMemcpyAsync(&flags, d_flags, sizeof(flags), cudaMemcpyDeviceToHost, ctx->stream));
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (flags & 1u) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_ckpt_decode_f32: character outside the base64 alphabet");
  if (flags & 2u) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_ckpt_decode_f32: malformed base64 padding");
  return VTLB_OK;
}
