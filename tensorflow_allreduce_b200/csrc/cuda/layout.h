// Constants and plain structs shared by host code and kernels: signal-pad layout and the
// per-rank synchronisation context handed to every collective kernel.
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace bc {
namespace dev {

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 512;     // barrier slots per channel
constexpr int kMetaBlocks = 64;     // blocks that may exchange per-call metadata (allgatherv)
constexpr int kUserChannels = 4;   // channels a caller can name: each has a stream, a signal pad and a staging slice
// A large staged allreduce of user channel c uses two more streams: c + kUserChannels, a second
// lane (stream and pad) on which every other chunk is reduced, so that the fixed costs of one
// reduction kernel (barriers, ramp-up, drain) hide behind the data phase of the other; and
// c + 2 * kUserChannels, on which the local copies into and out of the staging area run.
constexpr int kChannels = 3 * kUserChannels;

// Layout of one channel inside a rank's signal pad (all offsets in bytes).
constexpr size_t kFlagBytes = (size_t)kMaxBlocks * kMaxRanks * sizeof(uint32_t);          // 16 KiB
constexpr size_t kMetaBytes = (size_t)kMetaBlocks * kMaxRanks * 2 * sizeof(uint64_t);     // 16 KiB
// Progress words of the staged pipeline kernel: per peer and group of blocks one "chunks staged"
// and one "chunks reduced" counter, which only grow.
constexpr int kPipeMaxGroups = 8;
constexpr size_t kProgressBytes = 512;
constexpr size_t kChannelBytes = kFlagBytes + kMetaBytes + kProgressBytes;
constexpr size_t kPadBytes = kChannels * kChannelBytes;                                  // 390 KiB
constexpr int kPipeMaxChunks = 2048;   // chunks of one staged pipeline launch (local arrival counters: two per chunk)
static_assert(2 * kPipeMaxGroups * kMaxRanks * sizeof(uint32_t) <= kProgressBytes, "progress words do not fit");

// Status word written by a block whose wait ran out (host-mapped memory).
constexpr uint32_t kStatusTimeout = 0x80000000u;
// Status bit written by a bounds-checked build (-DBC_DEBUG) when an index left its tensor; the
// access is skipped, nothing traps.
constexpr uint32_t kStatusBounds = 0x40000000u;
// Status bit written when the ranks of an in-place reduction on symmetric memory did not all
// pass the same offset (the tensor is not at the same place on every rank).
constexpr uint32_t kStatusLayout = 0x20000000u;

// What one (real or emulated) rank needs to synchronise with its peers on one channel.
struct RankCtx {
  int rank;
  int world;
  uint32_t* flags[kMaxRanks];   // flags[p] = channel flag area inside rank p's pad
  uint64_t* meta[kMaxRanks];    // meta[p]  = channel metadata area inside rank p's pad
  uint32_t* epochs;             // this rank's private per-block epoch counters for the channel
  uint32_t* status;             // host-visible status word
  unsigned long long timeout_ns;
  // Barrier among the blocks of ONE rank's launch (kernels whose phases run on different numbers
  // of blocks): an arrival counter of this rank and channel in device memory, and its value
  // before this launch (the host adds up what every launch will contribute).
  uint32_t* local_ctr;
  uint32_t local_base;
};

}  // namespace dev
}  // namespace bc
