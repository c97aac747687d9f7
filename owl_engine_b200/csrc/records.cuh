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
}  // namespace owl
