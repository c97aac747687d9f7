// Slice-major record addressing shared by every kernel that reads a skinny record stream.
#pragma once
#include "common.cuh"

namespace owl {
constexpr int REC_SLICES = 8;
// Index (in records) of record (nt, kt) in a stream of NT x KT records stored
// [slice w][row tile][record of slice w], slice w = columns [w*KT/8, (w+1)*KT/8).
__host__ __device__ __forceinline__ size_t record_offset(int NT, int KT, int nt, int kt) {
  int w = (int)(((long long)(kt + 1) * REC_SLICES - 1) / KT);   // largest w with w*KT/8 <= kt
  int lo = (int)((long long)w * KT / REC_SLICES);
  if (lo > kt) { --w; lo = (int)((long long)w * KT / REC_SLICES); }
  const int hi = (int)((long long)(w + 1) * KT / REC_SLICES);
  return (size_t)NT * lo + (size_t)nt * (hi - lo) + (size_t)(kt - lo);
}
// Block-major stream: [128-row block][k-record][row tile of the block (8)], row tiles padded to a
// multiple of 8, so one (row block, k-record) block is 8 contiguous records and the k-records of
// a row block follow each other.
__host__ __device__ __forceinline__ size_t record_offset_block(int KT, int nt, int kt) {
  return ((size_t)(nt >> 3) * KT + kt) * 8 + (nt & 7);
}
// layout: 0 = slice-major, 1 = block-major
__host__ __device__ __forceinline__ size_t record_offset_any(int layout, int NT, int KT, int nt, int kt) {
  return layout ? record_offset_block(KT, nt, kt) : record_offset(NT, KT, nt, kt);
}
}  // namespace owl
