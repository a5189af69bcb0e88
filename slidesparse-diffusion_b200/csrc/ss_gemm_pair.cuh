// The sparse GEMM kernel: persistent clusters of two CTAs (tcgen05 cta_group::2).  Included by
// ss_gemm.cu inside namespace ss::{anonymous}, after KernelArgs, smem_desc and store_chunk.
//
// Why a pair: the two CTAs of a cluster compute 256 channels x N tokens together; each CTA loads,
// stores and reads its own 128 channel rows of A (compressed weights + metadata) and only HALF of
// the token rows of B (the hardware hands each half to the peer SM), which halves the dominant
// activation traffic per SM and per MMA.  That matters because a single CTA's sparse INT8 MMA is
// bound by the tensor core's 128 B/clk shared-memory read path, not by the tensor pipe (measured:
// ss_micro_mma_rate settles at 127.5 operand bytes per clock whatever N is; A is half as wide after
// compression, B is not).  No multicast load is involved.  What bounds the pair kernel is measured
// too, not assumed: first the two single threads that drive the pipeline (TMA issue, MMA
// issue, commits), now the round trip of the four-stage ring; see the diagnostics entry
// ss_micro_pair_rate and the counters a -DSS_TIMELINE build keeps.
//
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer (rank 0 only; also allocates TMEM), warps
// 2..9 epilogue (two per TMEM lane quadrant), warp 10 metadata copier (streaming form, rank 0).
//
// Protocol (rank = %cluster_ctarank):
//   full[s]      lives in rank 0 only.  Rank 0's producer posts the byte count of BOTH CTAs'
//                loads; both producers issue their loads with the cta_group::2 form, which
//                credits completion to rank 0's barrier; with a metadata warp its commit is the
//                barrier's second arrival.
//   empty[s]     one copy per CTA; the MMA thread (rank 0) commits with a 2-CTA multicast so
//                both producers see the stage free at the same time.
//   acc_full[b]  one copy per CTA, multicast commit; acc_empty[b] lives in rank 0 and counts the
//                16 epilogue warps of the pair (rank 1 arrives through shared::cluster).
// Every wait on these barriers is bounded (ptx::mbar_wait): a wait that runs out records the role
// in the device status word and the role winds down.
#pragma once

#ifndef SS_PAIR_EPI_WARPS
#define SS_PAIR_EPI_WARPS 8
#endif
constexpr int kPairEpiWarps = SS_PAIR_EPI_WARPS;       // 2 or 4 warps per TMEM lane quadrant
constexpr int kPairSub = kPairEpiWarps / 4;            // warps sharing a quadrant take chunks sub, sub+kPairSub, ...
// The last warp can issue the metadata copies (tcgen05.cp) so that the MMA thread, whose
// cta_group::2 operations cost about 125 cycles each to issue, only issues MMAs and commits
// (args.meta_warp).  It adds one barrier hop per stage, which pays with four or more pipeline
// stages (token tiles up to 224: -6 % on 4096x3072->9216) and costs with three (256).
constexpr int kPairThreads = 64 + 32 * kPairEpiWarps + 32;

// Per-tile time stamps of the three roles of each cluster's rank-0 CTA, for builds made with
// -DSS_TIMELINE only (a development aid; the shipped library does not contain it).
#ifdef SS_TIMELINE
constexpr int kTlTiles = 32, kTlSlots = 4, kTlClusters = 80;
__device__ long long g_timeline[kTlClusters * 3 * kTlTiles * kTlSlots];
#define SS_TL(role, tile_index, slot)                                                          \
  do {                                                                                         \
    if (rank == 0 && pair < kTlClusters && (tile_index) < kTlTiles)                            \
      g_timeline[((pair * 3 + (role)) * kTlTiles + (tile_index)) * kTlSlots + (slot)] = clock64(); \
  } while (0)
// per-cluster sums of the cycles the producer and the MMA thread spend in each kind of operation
constexpr int kPfSlots = 48;
__device__ long long g_profile[kTlClusters * kPfSlots];
#define SS_PF_BEGIN() long long pf_t = clock64()
#define SS_PF(acc) do { const long long pf_n = clock64(); (acc) += pf_n - pf_t; pf_t = pf_n; } while (0)
#define SS_PF_STORE(slot, value) do { if (rank == 0 && pair < kTlClusters) g_profile[pair * kPfSlots + (slot)] = (value); } while (0)
#else
#define SS_TL(role, tile_index, slot) do {} while (0)
#define SS_PF_BEGIN() do {} while (0)
#define SS_PF(acc) do {} while (0)
#define SS_PF_STORE(slot, value) do {} while (0)
#endif

// The pieces of work of a cluster, in order; a piece is the stages [s0, s1) of one tile (channel
// tile ch, token tile tok; tile = tok * tiles_ch2 + ch).
//   Whole-tile schedule: tiles pair, pair + clusters, ..., each with all its stages.  The two tile
//   indices are advanced without a division per tile (an integer division by a run-time value is a
//   chain of some 40 dependent instructions).
//   Split schedule (SPLIT): the launch's tiles x stages, in tile order, are cut into one contiguous
//   range per cluster, all of the same length to within one stage, so that no cluster idles in a
//   last partial round; a tile whose K extent is shared by several clusters is summed through
//   global memory (see the epilogue).
template <bool SPLIT>
struct Walk {
  int tile, ch, tok, s0, s1;
  bool valid;
  int step, step_ch, step_tok, tiles_ch2, num_st;
  long long pos, hi;
  __device__ __forceinline__ Walk(int pair, int num_pairs, int tiles_ch2_, int num_tiles, int num_st_)
      : tiles_ch2(tiles_ch2_), num_st(num_st_) {
    if constexpr (SPLIT) {
      const long long total = static_cast<long long>(num_tiles) * num_st;
      pos = pair * total / num_pairs;
      hi = (pair + 1) * total / num_pairs;
      step = step_ch = step_tok = 0;
      valid = pos < hi;
      decode();
    } else {
      tile = pair; ch = pair % tiles_ch2; tok = pair / tiles_ch2;
      step = num_pairs; step_ch = num_pairs % tiles_ch2; step_tok = num_pairs / tiles_ch2;
      s0 = 0; s1 = num_st; pos = 0; hi = num_tiles;
      valid = tile < num_tiles;
    }
  }
  __device__ __forceinline__ void decode() {
    tile = static_cast<int>(pos / num_st);
    s0 = static_cast<int>(pos - static_cast<long long>(tile) * num_st);
    const long long left = hi - pos;
    s1 = s0 + left < num_st ? s0 + static_cast<int>(left) : num_st;
    ch = tile % tiles_ch2;
    tok = tile / tiles_ch2;
  }
  __device__ __forceinline__ void advance() {
    if constexpr (SPLIT) {
      pos += s1 - s0;
      valid = pos < hi;
      if (valid) decode();
    } else {
      tile += step; ch += step_ch; tok += step_tok;
      if (ch >= tiles_ch2) { ch -= tiles_ch2; ++tok; }
      valid = tile < static_cast<int>(hi);
    }
  }
  __device__ __forceinline__ bool whole() const { return s0 == 0 && s1 == num_st; }
};

template <int NT, int KB>
struct PairTile {
  static constexpr int kHalf = NT / 2;                             // B token rows held per CTA
  static constexpr int kABytes = kTileCh * (kBlockK / 2) * KB;
  static constexpr int kBBlock = kHalf * kBlockK;
  static constexpr int kBBytes = kBBlock * KB;
  static constexpr int kEBlock = kTileCh * kBlockK / 8;
  static constexpr int kEBytes = kEBlock * KB;
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes;  // per CTA
  static constexpr int kStoreTile = 32 * 32 * 2;                    // 32 tokens x 32 channels BF16
  static constexpr int kBarBytes = 512;                             // barrier block
  static constexpr int kFixed = kBarBytes + 1024;                   // barrier block + alignment slack
  static constexpr int kBudget = 227 * 1024 - kFixed;
  // two staging tiles per epilogue warp if at least four pipeline stages still fit, else one
  static constexpr int kStages2 = (kBudget - 2 * kPairEpiWarps * kStoreTile) / kStageBytes;
  static constexpr int kStages1 = (kBudget - 1 * kPairEpiWarps * kStoreTile) / kStageBytes;
  static constexpr int kStoreBufs = kStages2 >= 4 ? 2 : 1;
  static constexpr int kStagesRaw = kStoreBufs == 2 ? kStages2 : kStages1;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kMetaColsPerStage = 4 * KB;
  static constexpr int kAccBufs = (kTmemCols - kStages * kMetaColsPerStage) / NT >= 2 ? 2 : 1;
  static constexpr int kMetaCol = kAccBufs * NT;
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + kStages * kABytes;
  static constexpr int kOffE = kOffB + kStages * kBBytes;
  static constexpr int kOffStore = kOffE + kStages * kEBytes;       // BF16 staging for TMA stores
  static constexpr int kOffBar = kOffStore + kStoreBufs * kPairEpiWarps * kStoreTile;
  static constexpr int kSmemBytes = kOffBar + kBarBytes + 1024;
  static_assert(kStages >= 2, "pipeline depth");
  static_assert(kMetaCol + kStages * kMetaColsPerStage <= kTmemCols, "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static_assert(NT % 16 == 0 && NT >= 64 && NT <= 256, "token tile of a CTA pair");
  // chunks of 32 tokens the epilogue walks; a tile of 240 ends in a half chunk of 16 tokens
  static constexpr int kChunks = (NT + 31) / 32;
  static constexpr bool kHalfTail = NT % 32 != 0;
  static_assert(kBBlock % 1024 == 0, "B blocks must keep the 128B-swizzle alignment");
};

// Output modes of the epilogue.
enum : int {
  kOutBf16 = 0,        // BF16, direct stores (any n, any alignment)
  kOutInt32 = 1,       // raw INT32 accumulators, direct stores
  kOutBf16Addend = 2,  // BF16 with an addend, direct stores
  kOutBf16Tma = 3,     // BF16 staged in shared memory and written with TMA tiled stores
  kOutBf16GateAdd = 4, // as kOutBf16Tma, but out += bf16(gate[batch, channel] * y) by TMA reduction
  kOutBf16TmaPeers = 5, // as kOutBf16Tma, but every tile is stored to several destinations (peer GPUs)
  kOutBf16TmaSplit = 6, // as kOutBf16Tma with the split schedule (see Walk): tiles may be shared by clusters
};

// Destination tensor maps of the tensor-parallel form; the other forms pass an empty struct.
struct PeerMaps { CUtensorMap m[kMaxPeers]; };

// Split schedule: words of the tile-sum area per epilogue warp (at most four 32 x 32 chunks) and
// per cluster (two CTAs of kPairEpiWarps warps).
constexpr int kSplitWarpWords = 4 * 1024;
constexpr long long kSplitClusterWords = 2ll * kPairEpiWarps * kSplitWarpWords;
struct NoPeers {};

// Shared-memory layout of the weights-resident form (RES): the whole K extent of the CTA's 128
// weight rows stays in shared memory (one slab per pipeline stage of K), the metadata of the whole
// K extent stays in TMEM, and the pipeline stages hold activations only.
template <int NT, int KB>
struct PairResident {
  using T = PairTile<NT, KB>;
  static constexpr int kMaxStagesK = (kTmemCols - 2 * NT) / T::kMetaColsPerStage;   // TMEM left for metadata
  static constexpr int kStoreBufs = 2;                              // staging tiles per epilogue warp
  static constexpr int kFixed = kStoreBufs * kPairEpiWarps * T::kStoreTile + T::kBarBytes + 1024;
  // kStages if that many B pipeline stages fit next to `slabs` resident A slabs, else 0
  static int b_stages(int slabs) {
    const int room = 227 * 1024 - kFixed - slabs * T::kABytes;
    const int stages = room / T::kBBytes;
    return stages < kStages ? 0 : kStages;
  }
  static constexpr int kStages = 4;     // activation stages of the resident form (the MMA loop is unrolled over them)
  static int smem_bytes(int slabs) { return slabs * T::kABytes + kStages * T::kBBytes + kFixed; }
};

template <int NT, int KB, int MODE, bool RES = false, class Peers = NoPeers>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
sparse_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_e,
                        const __grid_constant__ CUtensorMap map_out,
                        const __grid_constant__ CUtensorMap map_out_tail, const KernelArgs args,
                        const __grid_constant__ Peers peers) {
  using T = PairTile<NT, KB>;
  constexpr bool INT32_OUT = MODE == kOutInt32, HAS_ADDEND = MODE == kOutBf16Addend;
  constexpr bool SPLIT = MODE == kOutBf16TmaSplit;
  static_assert(!(SPLIT && RES), "the split schedule streams its weights");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int num_st = (args.num_kb + KB - 1) / KB;
  // pipeline depth and region offsets: compile-time in the streaming form, from the K extent in
  // the resident form (A slabs first, then the B stages, which also stage the metadata once)
  // pipeline depth: what fits in the streaming form, four activation stages in the resident form
  constexpr int kRing = RES ? PairResident<NT, KB>::kStages : T::kStages;
  constexpr int stages = kRing;
  const int off_a = 0;
  const int off_b = RES ? num_st * T::kABytes : T::kOffB;
  const int off_e = RES ? off_b : T::kOffE;
  const int off_store = RES ? off_b + stages * T::kBBytes : T::kOffStore;
  constexpr int kStoreBufs = RES ? PairResident<NT, KB>::kStoreBufs : T::kStoreBufs;
  const int off_bar = off_store + kStoreBufs * kPairEpiWarps * T::kStoreTile;
  constexpr int kBarStride = RES ? 8 : T::kStages;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + off_bar);
  uint64_t* bar_empty = bar_full + kBarStride;
  uint64_t* bar_acc_full = bar_empty + kBarStride;
  uint64_t* bar_acc_empty = bar_acc_full + T::kAccBufs;
  // streaming form: metadata of a stage is in TMEM (rank 0).  Resident form: [0] metadata of the
  // whole K extent is in TMEM (both CTAs), [1] resident operands have landed (rank 0)
  uint64_t* bar_meta = bar_acc_empty + T::kAccBufs;
  // streaming form: the metadata of a stage has landed in shared memory (rank 0).  It has a barrier
  // of its own so that its copy into TMEM runs while the stage's weights and activations still land.
  uint64_t* bar_e = bar_meta + kBarStride;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_e + kBarStride);
  static_assert((5 * kBarStride + 2 * T::kAccBufs) * 8 + 8 <= T::kBarBytes, "barrier block");
  static_assert(!RES || T::kAccBufs == 2, "resident form assumes two accumulators");
  static_assert(!(T::kHalfTail && MODE == kOutBf16TmaPeers), "the tensor-parallel stores take whole chunks only");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_ch2 = (args.tiles_ch + 1) >> 1;            // tiles of 256 channels
  const int num_tiles = tiles_ch2 * args.tiles_tok;
  const bool meta_warp = !RES && args.meta_warp != 0;
  // Tile sequence of this cluster: pair, pair + num_pairs, ...; tile = token tile * tiles_ch2 +
  // channel tile.  The resident form is launched with a cluster count that is a multiple of
  // tiles_ch2, so every tile of a cluster has the same channel tile (tile % tiles_ch2).
  const int tile_first = pair;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBarStride; ++s) {
      // a stage is ready when its operands have landed (the producer's arrival + the bytes) and, with
      // a metadata warp, when its metadata has been copied into TMEM (that warp's commit): one
      // barrier, so that the MMA thread polls once per stage
      ptx::mbar_init(&bar_full[s], meta_warp ? 2 : 1);
      ptx::mbar_init(&bar_empty[s], 1);
      ptx::mbar_init(&bar_meta[s], 1);
      ptx::mbar_init(&bar_e[s], 1);
    }
    for (int b = 0; b < T::kAccBufs; ++b) {
      ptx::mbar_init(&bar_acc_full[b], 1);
      ptx::mbar_init(&bar_acc_empty[b], 2 * kPairEpiWarps);
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_e);
    if constexpr (MODE == kOutBf16Tma || MODE == kOutBf16GateAdd || MODE == kOutBf16TmaSplit) {
      ptx::prefetch_tensormap(&map_out);
      if constexpr (T::kHalfTail) ptx::prefetch_tensormap(&map_out_tail);
    }
    if constexpr (MODE == kOutBf16TmaPeers) {
      for (int g = 0; g < args.peer_count; ++g) ptx::prefetch_tensormap(&peers.m[g]);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();            // the peer's barriers exist before anything is signalled there
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    // Three instructions per stage: the metadata and the activations as 3-D boxes whose outermost
    // coordinate is the block of 128 lifted columns (so that both blocks of a stage land back to
    // back), the weights as a box of both blocks side by side.  A box that reaches past the last
    // block is filled with zeros and still counts its full size on the barrier, so every stage
    // expects the same byte count.  Issuing a TMA instruction costs a thread 60 to 100 cycles, and
    // three lanes issuing one each in the same warp instruction cost the same as one lane issuing
    // three, so the count per stage is what matters: with five (one per 128-column block and
    // operand) this thread set the pace of the whole pipeline.
    if (lane == 0) {
      uint32_t s = 0, phase = 0;       // pipeline stage and the parity of its current use
      uint32_t issued = 0, tl = 0;     // stages filled so far
      bool ok = true;
      long long pf_wait = 0, pf_arm = 0, pf_a = 0, pf_b = 0, pf_e = 0;
      (void)pf_wait; (void)pf_arm; (void)pf_a; (void)pf_b; (void)pf_e;
      constexpr uint32_t kStageTx = 2u * (RES ? T::kBBytes : T::kABytes + T::kBBytes);   // both CTAs' bytes
      if constexpr (RES) {
        // the weights do not depend on the preceding kernel: fetch the resident operands first
        if (tile_first < num_tiles) {
          const int ch0 = (tile_first % tiles_ch2) * (2 * kTileCh) + static_cast<int>(rank) * kTileCh;
          if (rank == 0) ptx::mbar_arrive_expect_tx(&bar_meta[1], 2 * num_st * (T::kABytes + T::kEBytes));
          for (int st = 0; st < num_st; ++st) {
            ptx::tma_load_2d_pair(smem + off_a + st * T::kABytes, &map_a, &bar_meta[1], st * KB * (kBlockK / 2), ch0);
            // the metadata is staged where the first activation stages will live
            ptx::tma_load_3d_pair(smem + off_e + st * T::kEBytes, &map_e, &bar_meta[1], 0, ch0 >> 5, st * KB);
          }
          if (!ptx::mbar_wait(&bar_meta[0], 0, args.wait_ns)) ok = false;
        }
      }
      ptx::grid_dep_wait();           // q is written by the kernel launched just before this one
      for (Walk<SPLIT> w(pair, num_pairs, tiles_ch2, num_tiles, num_st); w.valid && ok; w.advance(), ++tl) {
        const int ch0 = w.ch * (2 * kTileCh) + static_cast<int>(rank) * kTileCh;
        const int tok0 = w.tok * NT + static_cast<int>(rank) * T::kHalf;
        SS_TL(0, tl, 0);
        for (int st = w.s0; st < w.s1; ++st) {
          SS_PF_BEGIN();
          if (!ptx::mbar_wait(&bar_empty[s], phase ^ 1u, args.wait_ns)) { ok = false; break; }
          SS_PF(pf_wait);
          if (rank == 0) {
            if constexpr (!RES) ptx::mbar_arrive_expect_tx(&bar_e[s], 2u * T::kEBytes);
            ptx::mbar_arrive_expect_tx(&bar_full[s], kStageTx);
          }
          SS_PF(pf_arm);
          if constexpr (!RES) {
            // the metadata first: it is small, and its copy into TMEM can start while the rest lands
            ptx::tma_load_3d_pair(smem + off_e + s * T::kEBytes, &map_e, &bar_e[s], 0, ch0 >> 5, st * KB);
            SS_PF(pf_e);
          }
          ptx::tma_load_3d_pair(smem + off_b + s * T::kBBytes, &map_b, &bar_full[s], 0, tok0, st * KB);
          SS_PF(pf_b);
          if constexpr (!RES) {
            ptx::tma_load_2d_pair(smem + off_a + s * T::kABytes, &map_a, &bar_full[s], st * KB * (kBlockK / 2), ch0);
            SS_PF(pf_a);
          }
          if (++s == static_cast<uint32_t>(kRing)) { s = 0; phase ^= 1u; }
          ++issued;
        }
        SS_TL(0, tl, 1);
      }
      SS_PF_STORE(0, pf_wait); SS_PF_STORE(1, pf_arm); SS_PF_STORE(2, pf_a); SS_PF_STORE(3, pf_b); SS_PF_STORE(4, pf_e);
      SS_PF_STORE(5, static_cast<long long>(issued));
      if (!ok) {
        atomicOr(args.status, kStatusProducerTimeout);
        // Let the copies already in flight land before the pair's shared memory is released.  The
        // full barriers live in rank 0 and count both CTAs' bytes, so rank 0 waits (bounded) for the
        // last fill of every stage that was filled; rank 1 is held by the cluster barrier at the end
        // of the kernel, which rank 0 reaches only after this loop.
        if (rank == 0) {
          const unsigned long long limit = args.wait_ns / 8 + 1;
          if constexpr (RES) ptx::mbar_wait(&bar_meta[1], 0, limit);
          for (uint32_t f = 0; f < static_cast<uint32_t>(kRing) && f < issued; ++f) {
            const uint32_t fills = (issued - f + kRing - 1) / kRing;
            ptx::mbar_wait(&bar_full[f], (fills - 1) & 1u, limit);
            if constexpr (!RES) ptx::mbar_wait(&bar_e[f], (fills - 1) & 1u, limit);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (rank 0 only)
    // The tensor pipe queues next to nothing: an MMA is accepted when the one before it is nearly
    // done, so whatever else this thread executes between two MMAs (address arithmetic, barrier
    // polls, commits) is time the pipe stands idle.  The ring is therefore unrolled with the stage
    // slot as a compile-time constant: every shared-memory descriptor is one add away from a
    // value computed before the loop, and a stage costs four MMAs, one commit and one barrier poll.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = (1u << 2) | (2u << 4) | (1u << 7) | (1u << 10) |
                                 (static_cast<uint32_t>(NT >> 3) << 17) |
                                 (static_cast<uint32_t>((2 * kTileCh) >> 4) << 24);
      constexpr uint32_t a_layout = KB == 2 ? 2u : 4u, a_sbo = KB == 2 ? 1024u : 512u;
      // descriptor = {low word: address / 16 | leading offset (16 B) / 16 << 16, high word: constant}
      constexpr uint32_t kDescHiA = (a_sbo >> 4) | (1u << 14) | (a_layout << 29);
      constexpr uint32_t kDescHiB = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t a_lo0 = ((ptx::smem_u32(smem + off_a) & 0x3ffffu) >> 4) | (1u << 16);
      const uint32_t b_lo0 = ((ptx::smem_u32(smem + off_b) & 0x3ffffu) >> 4) | (1u << 16);
      auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      const bool odd_tail = (args.num_kb % KB) != 0;       // the last stage of a tile holds one block only
      uint32_t phase = 0, acc_it = 0;
      bool ok = true;
      // diagnostics (ss_micro_pair_rate): cluster 0 reports the cycles its tile loop took; bit 0 of
      // args.debug leaves the MMAs out (commits only), so that the operand feed is timed alone
      const bool probe = args.probe != nullptr && pair == 0;
      const bool issue_mma = (args.debug & 1) == 0;
      long long probe_begin = 0;
      uint32_t probe_stages = 0, last_buf = 0, last_use = 0, tl = 0;
      long long pf_acc = 0, pf_ready = 0, pf_mma = 0, pf_commit = 0, pf_peek = 0;
      (void)pf_acc; (void)pf_ready; (void)pf_mma; (void)pf_commit; (void)pf_peek;
      Walk<SPLIT> w(pair, num_pairs, tiles_ch2, num_tiles, num_st);
      bool more = w.valid;
      if constexpr (RES) {
        // once per cluster: metadata of the whole K extent from its staging area into TMEM
        if (more) {
          if (!ptx::mbar_wait(&bar_meta[1], 0, args.wait_ns)) ok = false;
          ptx::tc_fence_after();
          const uint32_t e_addr = ptx::smem_u32(smem + off_e);
          const uint32_t e_tmem = tmem_base + T::kMetaCol;
          for (int kb = 0; kb < args.num_kb && ok; kb += 2) {
            if (kb + 1 < args.num_kb && args.wide_cp)
              ptx::tc_cp_128x256b_pair(e_tmem + 4 * kb, smem_desc(e_addr + kb * T::kEBlock, T::kEBlock, 128, 0));
            else
              for (int h = kb; h < kb + 2 && h < args.num_kb; ++h)
                ptx::tc_cp_128x128b_pair(e_tmem + 4 * h, smem_desc(e_addr + h * T::kEBlock, 128, 128, 0));
          }
          ptx::tc_commit_pair(&bar_meta[0], 3);       // both producers: the staging area is free
        }
      }
      if (probe) probe_begin = clock64();
      int st = w.s0, st_first = w.s0, st_end = w.s1;      // the current piece's stages
      uint32_t buf = 0, d_tmem = tmem_base;
      if (more && ok) {
        SS_TL(1, tl, 0);
        if (!ptx::mbar_wait(&bar_acc_empty[0], 1u, args.wait_ns)) ok = false;
        SS_TL(1, tl, 1);
        ptx::tc_fence_after();
      }
      while (more && ok) {
#pragma unroll
        for (int slot = 0; slot < kRing; ++slot) {
          SS_PF_BEGIN();
          if (!ptx::mbar_wait(&bar_full[slot], phase, args.wait_ns)) { ok = false; more = false; break; }
          if constexpr (!RES) {
            // without a metadata warp this thread copies the stage's metadata itself (below)
            if (!meta_warp && !ptx::mbar_wait(&bar_e[slot], phase, args.wait_ns)) { ok = false; more = false; break; }
          }
          SS_PF(pf_ready);
          if (st == st_first) SS_TL(1, tl, 2);
          ++probe_stages;
          ptx::tc_fence_after();
          // resident form: weights and metadata are indexed by the K position, not by the ring slot
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(RES ? st : slot) * (T::kABytes >> 4);
          const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(slot) * (T::kBBytes >> 4);
          const uint32_t e_tmem = tmem_base + T::kMetaCol + static_cast<uint32_t>(RES ? st : slot) * T::kMetaColsPerStage;
          const bool full_stage = !(odd_tail && st == num_st - 1);
          if (!RES && !meta_warp) {
            // no metadata warp (three pipeline stages): this thread copies the stage's metadata itself
            const uint32_t e_addr = ptx::smem_u32(smem + off_e) + slot * T::kEBytes;
            if (KB == 2 && full_stage && args.wide_cp) {
              // both metadata blocks of the stage in one instruction: block h is the h-th 16-byte
              // column of a 128 x 32-byte matrix whose columns lie kEBlock bytes apart
              ptx::tc_cp_128x256b_pair(e_tmem, smem_desc(e_addr, T::kEBlock, 128, 0));
            } else {
              for (int h = 0; h < (full_stage ? KB : 1); ++h)
                ptx::tc_cp_128x128b_pair(e_tmem + 4 * h, smem_desc(e_addr + h * T::kEBlock, 128, 128, 0));
            }
          }
          // K = 64 lifted columns per instruction: 32 B of compressed weights, 64 B of activations per row
          if (issue_mma) {
            ptx::tc_mma_sp_i8_pair(d_tmem, desc(a_lo, kDescHiA), desc(b_lo, kDescHiB), e_tmem, idesc, st != st_first ? 1u : 0u);
            ptx::tc_mma_sp_i8_pair(d_tmem, desc(a_lo + 2, kDescHiA), desc(b_lo + 4, kDescHiB), e_tmem + 2, idesc, 1u);
            if (KB == 2 && full_stage) {
              ptx::tc_mma_sp_i8_pair(d_tmem, desc(a_lo + 4, kDescHiA), desc(b_lo + (T::kBBlock >> 4), kDescHiB), e_tmem + 4, idesc, 1u);
              ptx::tc_mma_sp_i8_pair(d_tmem, desc(a_lo + 6, kDescHiA), desc(b_lo + (T::kBBlock >> 4) + 4, kDescHiB), e_tmem + 6, idesc, 1u);
            }
          }
          SS_PF(pf_mma);
          // The stage goes back to the producers as soon as its MMAs are queued (the arrival happens
          // when they have completed): the MMAs queue ahead of the pipe, so the commit costs this
          // thread time the pipe does not wait for, and the refill is not held up by the next
          // stage's arrival.
          ptx::tc_commit_pair(&bar_empty[slot], 3);
          SS_PF(pf_commit);
          if (slot == kRing - 1) phase ^= 1u;
          SS_PF(pf_peek);
          if (++st == st_end) {
            // the piece is complete: publish the accumulator
            ptx::tc_commit_pair(&bar_acc_full[buf], 3);
            SS_PF(pf_commit);
            SS_TL(1, tl, 3);
            last_buf = buf;
            last_use = acc_it / T::kAccBufs;
            w.advance();
            ++acc_it;
            ++tl;
            if (!w.valid) { more = false; break; }
            st = st_first = w.s0;
            st_end = w.s1;
            buf = acc_it % T::kAccBufs;
            d_tmem = tmem_base + buf * NT;
            SS_TL(1, tl, 0);
            if (!ptx::mbar_wait(&bar_acc_empty[buf], ((acc_it / T::kAccBufs) & 1u) ^ 1u, args.wait_ns)) { ok = false; more = false; break; }
            SS_PF(pf_acc);
            SS_TL(1, tl, 1);
            ptx::tc_fence_after();
          }
        }
      }
      SS_PF_STORE(8, pf_acc); SS_PF_STORE(9, pf_ready); SS_PF_STORE(10, pf_mma); SS_PF_STORE(11, pf_commit);
      SS_PF_STORE(12, pf_peek); SS_PF_STORE(13, static_cast<long long>(probe_stages));
      if (probe && ok && probe_stages > 0) {
        // the last tile's accumulator is complete when its barrier (this CTA's copy) flips
        if (!ptx::mbar_wait(&bar_acc_full[last_buf], last_use & 1u, args.wait_ns)) ok = false;
        args.probe[0] = static_cast<unsigned long long>(clock64() - probe_begin);
        args.probe[1] = probe_stages;
      }
      if (!ok) atomicOr(args.status, kStatusMmaTimeout);
    }
  } else if (warp == 2 + kPairEpiWarps) {
    // ------------------------------------------------------------------ metadata copier (rank 0 only)
    if (meta_warp && lane == 0 && rank == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (Walk<SPLIT> w(pair, num_pairs, tiles_ch2, num_tiles, num_st); w.valid && ok; w.advance()) {
        for (int st = w.s0; st < w.s1; ++st) {
          const int kb0 = st * KB;
          const int nkb = args.num_kb - kb0 < KB ? args.num_kb - kb0 : KB;
          // the stage's previous metadata is no longer read once its MMAs have completed, which
          // the producer has already waited for before refilling the stage
          if (!ptx::mbar_wait(&bar_e[s], phase, args.wait_ns)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t e_addr = ptx::smem_u32(smem + off_e + s * T::kEBytes);
          const uint32_t e_tmem = tmem_base + T::kMetaCol + s * T::kMetaColsPerStage;
          if (KB == 2 && nkb == 2 && args.wide_cp) {
            // both metadata blocks of the stage in one instruction: block h is the h-th 16-byte
            // column of a 128 x 32-byte matrix whose columns lie kEBlock bytes apart
            ptx::tc_cp_128x256b_pair(e_tmem, smem_desc(e_addr, T::kEBlock, 128, 0));
          } else {
            for (int h = 0; h < nkb; ++h)
              ptx::tc_cp_128x128b_pair(e_tmem + 4 * h, smem_desc(e_addr + h * T::kEBlock, 128, 128, 0));
          }
          ptx::tc_commit_pair(&bar_full[s], 1);      // arrives (rank 0 only) when the copy has completed
          if (++s == static_cast<uint32_t>(kRing)) { s = 0; phase ^= 1u; }
        }
      }
      if (!ok) atomicOr(args.status, kStatusMmaTimeout);
    }
  } else if constexpr (MODE == kOutBf16Tma || MODE == kOutBf16GateAdd || MODE == kOutBf16TmaPeers || MODE == kOutBf16TmaSplit) {
    // ------------------------------------------------------------------ epilogue, TMA stores
    constexpr bool GATED = MODE == kOutBf16GateAdd;
    // The accumulator is channel-major in TMEM (lane = channel, column = token) and the output is
    // token-major.  tcgen05.ld in the 16x256b fragment layout hands each thread two adjacent
    // tokens of one channel per register pair, which is exactly what stmatrix.trans needs to
    // write 8 tokens x 8 channels blocks token-major: two values are converted with one packed
    // BF16 conversion and 32 of them stored with one stmatrix.x4.
    // Token scales never touch shared memory: lane l keeps the scale of token l of each of the
    // warp's chunks in a register (fetched one tile ahead) and the lanes exchange them by shuffle.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;             // this warp takes chunks half, half + kPairSub, ...
    const int lane_ch = lane >> 2, tpair = (lane & 3) * 2;
    uint32_t acc_it = 0, store_it = 0, tl = 0;
    bool ok = true;
    const bool tl_warp = warp == 2 && lane == 0;
    constexpr int kMine = (T::kChunks + kPairSub - 1) / kPairSub;     // chunks per warp and tile, at most
    float sa_next[kMine], sw_next[4], bias_next[4];
#ifdef SS_TIMELINE
    long long pe_acc = 0, pe_ld = 0, pe_prep = 0, pe_math = 0, pe_fence = 0, pe_store = 0, pe_rest = 0, pe_chunks = 0, pe_commit = 0, pe_null = 0, pe_reconv = 0;
#endif
    // The scales of the next tile are fetched while this one is processed.  The loads must not be
    // consumed where they are issued (a select on the loaded value would wait an L2 round trip
    // here, once per tile): indices are clamped into range instead, and what a lane then holds
    // for a token >= m or a channel >= n multiplies values that the stores clip.
#pragma unroll
    for (int i = 0; i < 4; ++i) bias_next[i] = 0.f;
    const int last_tok = args.m - 1, last_ch = args.n - 1;
    Walk<SPLIT> nxt(pair, num_pairs, tiles_ch2, num_tiles, num_st);
    auto prefetch = [&]() {
      const int pch = nxt.ch * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32 + lane_ch;
      const int ptok = nxt.tok * NT + half * 32 + lane;
#pragma unroll
      for (int i = 0; i < kMine; ++i) sa_next[i] = __ldg(args.sa + min(ptok + kPairSub * 32 * i, last_tok));
#pragma unroll
      for (int i = 0; i < 4; ++i) sw_next[i] = __ldg(args.sw + min(pch + 8 * i, last_ch));   // channels lane_ch + 8 i
      if (args.bias) {
#pragma unroll
        for (int i = 0; i < 4; ++i) bias_next[i] = __ldg(args.bias + min(pch + 8 * i, last_ch));
      }
    };
    ptx::grid_dep_wait();             // sa is written by the kernel launched just before this one
    if (nxt.valid) prefetch();
    for (; nxt.valid && ok; ++acc_it, ++tl) {
      const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
      const int ch_w = nxt.ch * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32;
      const int tok0 = nxt.tok * NT;
      // Split schedule: a tile whose stages are shared by several clusters (`pieces` of them, the
      // first being cluster `owner`) is completed through global memory: every piece but the last to
      // arrive stores its accumulator in a slab of its own, and the last one adds them up and runs
      // the epilogue (integer addition is exact, so the order of arrival does not matter, and nobody
      // waits for anybody).  A cluster has two slabs: one for a piece that starts its tile (`head`:
      // the last piece of the cluster's range) and one for a piece that does not (the first piece of
      // its range).  Cluster c works on positions [c * total / clusters, (c + 1) * total / clusters)
      // of the tiles x stages sequence, so position P belongs to cluster
      // ceil((P + 1) * clusters / total) - 1.
      bool partial = false, head = false;
      int pieces = 1, owner = 0;
      int* counter = nullptr;
      if constexpr (SPLIT) {
        partial = !nxt.whole();
        if (partial) {
          const long long total = static_cast<long long>(num_tiles) * num_st;
          const long long first = static_cast<long long>(nxt.tile) * num_st;
          owner = static_cast<int>(((first + 1) * num_pairs + total - 1) / total) - 1;
          pieces = static_cast<int>(((first + num_st) * num_pairs + total - 1) / total) - owner;
          head = nxt.s0 == 0;
          counter = args.split_ticket + owner * (2 * kPairEpiWarps) + static_cast<int>(rank) * kPairEpiWarps + (warp - 2);
        }
      }
      // this warp's part of a slab: chunk i, registers 4 g .. 4 g + 3 of lane l at uint4 (8 i + g) * 32 + l
      auto slab = [&](int cluster, bool of_head) {
        const long long slot = (static_cast<long long>(cluster) * 2 + (of_head ? 0 : 1)) * (2 * kPairEpiWarps) +
                               static_cast<int>(rank) * kPairEpiWarps + (warp - 2);
        return reinterpret_cast<uint4*>(args.split_sum) + slot * (kSplitWarpWords / 4) + lane;
      };
      float sa_mine[kMine], sw[4], bias[4];
#pragma unroll
      for (int i = 0; i < kMine; ++i) sa_mine[i] = sa_next[i];
#pragma unroll
      for (int i = 0; i < 4; ++i) { sw[i] = sw_next[i]; bias[i] = bias_next[i]; }
      nxt.advance();
      if (nxt.valid) prefetch();
      int chunks = (args.m - tok0 + 31) / 32;
      chunks = chunks < T::kChunks ? chunks : T::kChunks;
      const int mine = chunks > half ? (chunks - half + kPairSub - 1) / kPairSub : 0;
      uint32_t f[2][32];
      // split schedule: this warp's chunk i of a slab into registers
      auto fetch = [&](uint32_t (&r)[32], const uint4* src, int i) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint4 v = __ldcg(src + (8 * i + g) * 32);
          r[4 * g] = v.x; r[4 * g + 1] = v.y; r[4 * g + 2] = v.z; r[4 * g + 3] = v.w;
        }
      };
      // are all the other pieces of the tile in?
      auto others_in = [&]() {
        int seen = 0;
        if (lane == 0) seen = atomicAdd(counter, 0);
        const bool all = __shfl_sync(0xffffffffu, seen, 0) == pieces - 1;
        if (all) __threadfence();
        return all;
      };
      // A head piece ends its cluster's range, the others start theirs, so the head piece is nearly
      // always the last to arrive.  It looks while its own MMAs still run; if the others are all in
      // it starts fetching the next cluster's slab now and later adds the slabs to its accumulator
      // as that leaves TMEM, instead of storing and re-reading it.
      bool finish = false, primed = false;
      if constexpr (SPLIT) {
        if (partial && head && mine > 0 && !(args.debug & 2)) {
          finish = others_in();
          if (finish) { fetch(f[1], slab(owner + 1, false), 0); primed = true; }
        }
      }
      if (tl_warp) SS_TL(2, tl, 0);
      SS_PF_BEGIN();
      if (!ptx::mbar_wait(&bar_acc_full[buf], acc_use & 1u, args.wait_ns)) { ok = false; break; }
      SS_PF(pe_acc);
      if (tl_warp) SS_TL(2, tl, 1);
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * NT;
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_rank0(&bar_acc_empty[buf]);
        if (tl_warp) SS_TL(2, tl, 2);
      };
      if (args.debug & 2) {          // diagnostics: main loop alone, the accumulator is handed straight back
        release();
        continue;
      }
      auto load = [&](uint32_t (&f)[32], int c) {
        ptx::tc_ld_16x256b_x4(t_addr + c * 32, f);                       // channels 0..15 of the quadrant
        ptx::tc_ld_16x256b_x4(t_addr + (16u << 16) + c * 32, f + 16);    // channels 16..31
      };
      auto emit = [&](const uint32_t (&f)[32], int c, float sa_lane) {
        uint8_t* stage = smem + off_store + ((warp - 2) * kStoreBufs + (store_it % kStoreBufs)) * T::kStoreTile;
        // scales of this thread's eight tokens (8 g + tpair, + 1), from the lanes that hold them
        float2 sa_tok[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          sa_tok[g].x = __shfl_sync(0xffffffffu, sa_lane, 8 * g + tpair);
          sa_tok[g].y = __shfl_sync(0xffffffffu, sa_lane, 8 * g + tpair + 1);
        }
        if (lane == 0) {
          // the staging tile about to be rewritten: its last store must have finished reading it
          if constexpr (kStoreBufs == 2) ptx::bulk_wait_read<1>(); else ptx::bulk_wait_read<0>();
        }
        __syncwarp();
        SS_PF(pe_prep);
        // gated accumulation: the 32 tokens of a chunk belong to one batch (rows_per_batch % 32 == 0)
        float gate[4] = {1.f, 1.f, 1.f, 1.f};
        if constexpr (GATED) {
          const __nv_bfloat16* g = args.gate + static_cast<long long>((tok0 + c * 32) / args.rows_per_batch) * args.gate_stride;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int ch = ch_w + lane_ch + 8 * i;
            gate[i] = ch < args.n ? __bfloat162float(g[ch]) : 0.f;
          }
        }
        // this thread addresses row lane%8 of matrix lane/8 in every stmatrix.x4: matrices are
        // (token group, channel group) = (2 gp, 2 h), (2 gp, 2 h + 1), (2 gp + 1, 2 h), (2 gp + 1, 2 h + 1);
        // rows are 64 bytes (32 channels) with the 16-byte pieces XOR-swizzled as TMA's 64B mode expects
        const int mi = lane >> 3;
        const uint32_t stage_addr = ptx::smem_u32(stage);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int gp = 0; gp < 2; ++gp) {
            uint32_t packed[4];
#pragma unroll
            for (int gi = 0; gi < 2; ++gi) {
              const int g = 2 * gp + gi;
              const float2 s = sa_tok[g];                                    // tokens 8 g + tpair, + 1
              const uint32_t* r = f + 16 * h + 4 * g;
#pragma unroll
              for (int ab = 0; ab < 2; ++ab) {
                // two tokens of one channel at a time with the packed FP32 instructions: each half is
                // the same IEEE multiply / fused multiply-add (round to nearest) as the scalar form
                const float w = sw[2 * h + ab], b = bias[2 * h + ab];
                const float2 acc = make_float2(__int2float_rn(static_cast<int32_t>(r[2 * ab])),
                                               __int2float_rn(static_cast<int32_t>(r[2 * ab + 1])));
                float2 y = __ffma2_rn(acc, __fmul2_rn(s, make_float2(w, w)), make_float2(b, b));
                if constexpr (GATED) y = __fmul2_rn(make_float2(gate[2 * h + ab], gate[2 * h + ab]), y);
                const __nv_bfloat162 p = __floats2bfloat162_rn(y.x, y.y);   // low half = even token
                packed[2 * gi + ab] = *reinterpret_cast<const uint32_t*>(&p);
              }
            }
            const int tok = 8 * (2 * gp + (mi >> 1)) + (lane & 7);
            const int cg = 2 * h + (mi & 1);
            ptx::stmatrix_x4_trans(stage_addr + tok * 64 + ((cg ^ ((tok >> 1) & 3)) << 4),
                                   packed[0], packed[1], packed[2], packed[3]);
          }
        }
        SS_PF(pe_math);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        SS_PF(pe_fence);
        if (lane == 0) {
          // rows >= m and channels >= n are clipped by the tensor map; a box that lies wholly
          // beyond the last channel is not issued at all
          // the half chunk that ends a 240-token tile goes out through a 16-token box: the other 16
          // staged rows hold columns of the neighbouring accumulator and belong to the next tile
          const CUtensorMap* dst = (T::kHalfTail && c == T::kChunks - 1) ? &map_out_tail : &map_out;
          if (ch_w < args.n && !(args.debug & 4)) {
            if constexpr (GATED) {
              ptx::tma_reduce_add_2d(dst, stage, ch_w, tok0 + c * 32);
            } else if constexpr (MODE == kOutBf16TmaPeers) {
              // the same staged tile goes to this GPU's and every peer's gathered output
              for (int g = 0; g < args.peer_count; ++g) ptx::tma_store_2d(&peers.m[g], stage, ch_w, tok0 + c * 32);
            } else if (args.out_evict_first) {
              ptx::tma_store_2d_evict_first(dst, stage, ch_w, tok0 + c * 32);
            } else {
              ptx::tma_store_2d(dst, stage, ch_w, tok0 + c * 32);
            }
          }
          SS_PF(pe_store);
          ptx::bulk_commit();
          SS_PF(pe_commit);
          SS_PF(pe_null);
        }
        SS_PF(pe_reconv);
        ++store_it;
      };
      if (mine == 0) {
        release();
      } else if (SPLIT && partial) {
        auto add_pieces = [&](int first_piece, int i) {       // f[0] += pieces first_piece .. of chunk i
          for (int p = first_piece; p < pieces; ++p) {
            fetch(f[1], slab(owner + p, p == 0), i);
#pragma unroll
            for (int j = 0; j < 32; ++j) f[0][j] += f[1][j];
          }
        };
        if (head && !finish) finish = others_in();
        if (finish && !primed) fetch(f[1], slab(owner + 1, false), 0);
        uint4* own = slab(pair, head);
#pragma unroll
        for (int i = 0; i < kMine; ++i) {
          if (i < mine) {
            const int c = half + kPairSub * i;
            load(f[0], c);
            ptx::tc_wait_ld();
            if (i + 1 == mine) release();
            if (finish) {
              // the next cluster's slab (fetched during the previous chunk's emit), then any further ones
#pragma unroll
              for (int j = 0; j < 32; ++j) f[0][j] += f[1][j];
              add_pieces(2, i);
              if (i + 1 < mine) fetch(f[1], slab(owner + 1, false), i + 1);
              emit(f[0], c, sa_mine[i]);
            } else {
#pragma unroll
              for (int g = 0; g < 8; ++g)
                __stcg(own + (8 * i + g) * 32, make_uint4(f[0][4 * g], f[0][4 * g + 1], f[0][4 * g + 2], f[0][4 * g + 3]));
            }
          }
        }
        if (!finish) {
          __threadfence();                  // this lane's stores before the ticket
          __syncwarp();
          int ticket = 0;
          if (lane == 0) ticket = atomicAdd(counter, 1);
          finish = __shfl_sync(0xffffffffu, ticket, 0) == pieces - 1;
          if (finish) {
            __threadfence();
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
              if (i < mine) {
                fetch(f[0], slab(owner, true), i);
                add_pieces(1, i);
                emit(f[0], half + kPairSub * i, sa_mine[i]);
              }
            }
          }
        }
        if (finish && lane == 0) atomicExch(counter, 0);      // zero between launches
      } else {
        load(f[0], half);
#pragma unroll
        for (int i = 0; i < kMine; ++i) {
          if (i < mine) {
            const int c = half + kPairSub * i;
            SS_PF(pe_rest);
            ptx::tc_wait_ld();
            // The accumulator goes back to the MMA thread as soon as its last chunk is in registers:
            // when the load issued here is the last one it is waited for at once (its latency, some
            // 80 cycles, is then not hidden behind an emit) and the buffer is released a whole emit
            // earlier.  With few stages per tile the MMA thread otherwise waits for this release.
            if (i + 1 < mine) load(f[(i + 1) & 1], c + kPairSub);
            if (i + 2 == mine) { ptx::tc_wait_ld(); release(); }
            else if (mine == 1) release();
            SS_PF(pe_ld);
            if (!(args.debug & 8)) emit(f[i & 1], c, sa_mine[i]);
#ifdef SS_TIMELINE
            ++pe_chunks;
#endif
          }
        }
      }
      if (tl_warp) SS_TL(2, tl, 3);
#ifdef SS_TIMELINE
      if (tl_warp && tl == 0) {        // the first tile's sums on their own
        SS_PF_STORE(32, pe_acc); SS_PF_STORE(33, pe_ld); SS_PF_STORE(34, pe_prep); SS_PF_STORE(35, pe_math);
        SS_PF_STORE(36, pe_fence); SS_PF_STORE(37, pe_store); SS_PF_STORE(38, pe_rest); SS_PF_STORE(39, pe_chunks);
        SS_PF_STORE(40, pe_commit); SS_PF_STORE(41, pe_reconv);
      }
#endif
    }
    if (lane == 0) ptx::bulk_wait_all();
    __syncwarp();
#ifdef SS_TIMELINE
    if (tl_warp) {
      SS_PF_STORE(16, pe_acc); SS_PF_STORE(17, pe_ld); SS_PF_STORE(18, pe_prep); SS_PF_STORE(19, pe_math);
      SS_PF_STORE(20, pe_fence); SS_PF_STORE(21, pe_store); SS_PF_STORE(22, pe_rest); SS_PF_STORE(23, pe_chunks);
      SS_PF_STORE(24, pe_commit); SS_PF_STORE(25, pe_null); SS_PF_STORE(26, pe_reconv);
    }
#endif
    if (!ok && lane == 0) atomicOr(args.status, kStatusEpilogueTimeout);
  } else {
    // ------------------------------------------------------------------ epilogue, direct stores
    // (unaligned output, addend, INT32 dump): lane = channel, 32 token columns per tcgen05.ld
    const int quad = warp & 3;                    // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;             // which of the quadrant's warps: chunks half, half+kPairSub, ...
    uint32_t acc_it = 0;
    bool ok = true;
    // Scales of a tile are fetched one tile ahead into registers (the loads fly while the previous
    // tile is processed): lane l holds the scale of token l of each of the warp's chunks.
    constexpr int kMine = (T::kChunks + kPairSub - 1) / kPairSub;
    float sa_next[kMine], sw_next = 1.f, bias_next = 0.f;
    // indices clamped into range rather than loads under a condition: see the TMA-store epilogue
    const int last_tok = args.m - 1, last_ch = args.n - 1;
    Walk<false> nxt(pair, num_pairs, tiles_ch2, num_tiles, num_st);
    auto prefetch = [&]() {
      const int pch = nxt.ch * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32 + lane;
      const int ptok = nxt.tok * NT + half * 32 + lane;
#pragma unroll
      for (int i = 0; i < kMine; ++i) sa_next[i] = __ldg(args.sa + min(ptok + kPairSub * 32 * i, last_tok));
      sw_next = __ldg(args.sw + min(pch, last_ch));
      if (args.bias) bias_next = __ldg(args.bias + min(pch, last_ch));
    };
    ptx::grid_dep_wait();
    if constexpr (!INT32_OUT) {
      if (nxt.valid) prefetch();
    }
    for (; nxt.valid && ok; ++acc_it) {
      const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
      const int ch = nxt.ch * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32 + lane;
      const int tok0 = nxt.tok * NT;
      const bool ch_ok = ch < args.n;
      float sa_mine[kMine], sw = 1.f, bias = 0.f;
#pragma unroll
      for (int i = 0; i < kMine; ++i) sa_mine[i] = 1.f;
      nxt.advance();
      if constexpr (!INT32_OUT) {
#pragma unroll
        for (int i = 0; i < kMine; ++i) sa_mine[i] = sa_next[i];
        sw = sw_next;
        bias = bias_next;
        if (nxt.valid) prefetch();
      }
      int chunks = (args.m - tok0 + 31) / 32;
      chunks = chunks < T::kChunks ? chunks : T::kChunks;
      if (!ptx::mbar_wait(&bar_acc_full[buf], acc_use & 1u, args.wait_ns)) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * NT;
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_rank0(&bar_acc_empty[buf]);
      };
      if (args.debug & 2) {
        release();
        continue;
      }
      const int tok_end = tok0 + NT < args.m ? tok0 + NT : args.m;
      const int mine = chunks > half ? (chunks - half + kPairSub - 1) / kPairSub : 0;
      if (mine == 0) {
        release();
      } else {
        uint32_t r[2][32];
        ptx::tc_ld_32x32b_x32(t_addr + half * 32, r[0]);
#pragma unroll
        for (int i = 0; i < kMine; ++i) {
          if (i < mine) {
            const int c = half + kPairSub * i;
            ptx::tc_wait_ld();
            // as in the TMA-store epilogue: the last load is waited for where it is issued, so that
            // the accumulator is released before the last two chunks are stored
            if (i + 1 < mine) ptx::tc_ld_32x32b_x32(t_addr + (c + kPairSub) * 32, r[(i + 1) & 1]);
            if (i + 2 == mine) { ptx::tc_wait_ld(); release(); }
            else if (mine == 1) release();
            store_chunk<INT32_OUT, HAS_ADDEND>(r[i & 1], args, sa_mine[i], tok0 + c * 32, tok_end, ch, ch_ok, sw, bias);
          }
        }
      }
    }
    if (!ok && lane == 0) atomicOr(args.status, kStatusEpilogueTimeout);
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();            // neither CTA leaves while the peer may still touch its memory
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}
