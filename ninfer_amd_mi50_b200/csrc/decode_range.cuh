// The key range of one decode row, shared by the kernels of attention_decode.cu and
// attention_decode_stream.cu so that they agree on which blocks of 128 keys a row has.
#pragma once

namespace nf {

// Row at position `pos` with `window` (0: none) and a workspace of `nsplit` blocks of `block`
// keys: sets lo..pos to the keys the row reads.  A position that needs a block beyond the
// workspace is cut to the workspace's last key (and lo to at most that), so that every block in
// [lo / block, pos / block] exists and holds a key; returns true when it had to cut.
__device__ __forceinline__ bool decode_key_range(int& pos, int& lo, int window, int nsplit, int block) {
  lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int most = nsplit * block - 1;
  if (pos <= most) return false;
  pos = most;
  if (lo > pos) lo = pos;
  return true;
}

}  // namespace nf
