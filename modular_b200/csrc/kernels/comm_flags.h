// Word layout of a rank's tensor-parallel flag array (int32, symmetric memory, zeroed once).
// Shared by the communication kernels (comm.cu) and the GEMMs that are fused with a collective
// (gemm_comm.cu).
//
//   [slot * 8 + src]  slot 0..3   barrier words: rank `src` writes its epoch here on every peer
//   kEpochWord        barrier epoch of this rank (advanced by the kernels themselves, so captured
//                     CUDA graphs replay with fresh epochs)
//   kDoneWord         CTAs of the running communication kernel that finished their part
//   kReady + src      "rows of rank src have landed in your activation buffer" epoch (remote write)
//   kReadyEpoch       how many signalling reduce+norm kernels this rank has run (local)
//   kPushTarget       value kPushCount reaches once all partial tiles of the current GEMM landed
//   kPushCount        partial tiles that have landed here (one remote add per source rank and GEMM)
//   kPushLocal + o    local count of this rank's GEMM CTAs that finished a tile destined for owner o
#pragma once

namespace mb {

constexpr int kMaxRanks = 8;
constexpr int kFlagSlots = 4;
constexpr int kEpochWord = kFlagSlots * kMaxRanks;  // 32
constexpr int kDoneWord = kEpochWord + 1;           // 33
constexpr int kReady = 40;                          // 40..47
constexpr int kReadyEpoch = 48;
constexpr int kPushTarget = 49;
constexpr int kPushCount = 64;                      // on a cache line of its own
constexpr int kPushLocal = 72;                      // 72..79: tiles of the running GEMM finished per owner
constexpr int kTpFlagInts = 96;

// State words of the decode GEMM (gemm_decode.cu), local device memory, zeroed once:
//   kDecArrive        CTAs of the running kernel whose partial tiles are written
//   kDecDepart        CTAs that have left; the last one clears both counters
//   kDecGen           all-reduce generation (advanced by the kernel, so graph replays stay in step)
//   kDecGenRows + i   token rows written into receive-buffer generation i the last time it was used
constexpr int kDecArrive = 0;
constexpr int kDecDepart = 1;
constexpr int kDecGen = 2;
constexpr int kDecGenRows = 3;                      // 3..5
//   kDecTileCnt + j   contributors of output tile (or gate / up tile pair) j that have written their partial; the
//                     one that completes the count runs the tile's epilogue and clears the word
constexpr int kDecTileCnt = 8;
constexpr int kDecTileCounters = 4096;
constexpr int kDecStateInts = kDecTileCnt + kDecTileCounters;

}  // namespace mb
