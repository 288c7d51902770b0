// Work items of the paged decode: one 64-bit word per 256-token chunk of one query head.
//
//   bits  0.. 8  tokens in this chunk (0 = empty slot, skipped)
//   bits  9..21  chunk index within the head
//   bits 22..35  number of chunks of the head
//   bits 36..55  flat query-head index (b * H_q + h)
//
// Selection kernels emit the list; the decode kernels' persistent blocks walk it.
#pragma once

#include "ekv_common.cuh"

namespace ekv {

constexpr int kItemMaxChunks = 1 << 13;   // 8192 chunks = 2M tokens per head
constexpr int kItemMaxHeads = 1 << 20;

__host__ __device__ inline unsigned long long make_item(int head, int chunk, int head_tokens) {
  const int nch = (head_tokens + kChunkTokens - 1) / kChunkTokens;
  int ntok = head_tokens - chunk * kChunkTokens;
  ntok = ntok < 0 ? 0 : (ntok > kChunkTokens ? kChunkTokens : ntok);
  return (unsigned long long)ntok | ((unsigned long long)chunk << 9) | ((unsigned long long)nch << 22) |
         ((unsigned long long)head << 36);
}
__host__ __device__ inline int item_ntok(unsigned long long d) { return (int)(d & 0x1ffu); }
__host__ __device__ inline int item_chunk(unsigned long long d) { return (int)((d >> 9) & 0x1fffu); }
__host__ __device__ inline int item_nch(unsigned long long d) { return (int)((d >> 22) & 0x3fffu); }
__host__ __device__ inline int item_head(unsigned long long d) { return (int)((d >> 36) & 0xfffffu); }

}  // namespace ekv
