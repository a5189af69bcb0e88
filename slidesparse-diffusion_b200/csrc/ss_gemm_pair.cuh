// CTA-pair variant of the sparse GEMM (tcgen05 cta_group::2).  Included by ss_gemm.cu inside
// namespace ss::{anonymous}, after KernelArgs, smem_desc, mbar_peek and store_chunk.
//
// Why a pair: the single-CTA kernel is bound by shared-memory bandwidth, not by the tensor
// pipe.  A K=64 sparse INT8 MMA of M=128 x N reads 4 KB of A and 64*N bytes of B from shared
// memory, and TMA wrote the same bytes there a moment earlier; at 128 B/clk for reads and writes
// together that is 2*(5 KB + 64*N) / 128 cycles against N/2 cycles of tensor work (36 % of the
// tensor peak at N = 192).  With cta_group::2 the two CTAs of a cluster compute 256 channels x N
// tokens together: each CTA stores and reads its own 128 channel rows of A and only HALF of the
// token rows of B (the hardware hands each half to the peer SM), which halves the dominant B
// traffic (61 % at N = 256, 58 % at N = 224).  No multicast load is involved.
//
// Protocol (rank = %cluster_ctarank):
//   full[s]      lives in rank 0 only.  Rank 0's producer posts the byte count of BOTH CTAs'
//                loads; both producers issue their loads with the cta_group::2 form, which
//                credits completion to rank 0's barrier.
//   empty[s]     one copy per CTA; the MMA thread (rank 0) commits with a 2-CTA multicast so
//                both producers see the stage free at the same time.
//   acc_full[b]  one copy per CTA, multicast commit; acc_empty[b] lives in rank 0 and counts the
//                8 epilogue warps of the pair (rank 1 arrives through shared::cluster).
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

template <int NT, int KB>
struct PairTile {
  static constexpr int kHalf = NT / 2;                             // B token rows held per CTA
  static constexpr int kABytes = kTileCh * (kBlockK / 2) * KB;
  static constexpr int kBBlock = kHalf * kBlockK;
  static constexpr int kBBytes = kBBlock * KB;
  static constexpr int kEBlock = kTileCh * kBlockK / 8;
  static constexpr int kEBytes = kEBlock * KB;
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes;  // per CTA
  static constexpr int kSaBytes = kPairEpiWarps * NT * 4;           // token scales, one copy per warp
  static constexpr int kStoreTile = 32 * 32 * 2;                    // 32 tokens x 32 channels BF16
  static constexpr int kFixed = kSaBytes + 256 + 1024;              // + barrier block + alignment slack
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
  static constexpr int kOffSa = kOffE + kStages * kEBytes;
  static constexpr int kOffStore = kOffSa + kSaBytes;               // BF16 staging for TMA stores
  static constexpr int kOffBar = kOffStore + kStoreBufs * kPairEpiWarps * kStoreTile;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;
  static_assert(kStages >= 2, "pipeline depth");
  static_assert(kMetaCol + kStages * kMetaColsPerStage <= kTmemCols, "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static_assert(NT % 32 == 0 && NT >= 64 && NT <= 256, "token tile of a CTA pair");
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
};

// Destination tensor maps of the tensor-parallel form; the other forms pass an empty struct.
struct PeerMaps { CUtensorMap m[kMaxPeers]; };
struct NoPeers {};

// Shared-memory layout of the weights-resident form (RES): the whole K extent of the CTA's 128
// weight rows stays in shared memory (one slab per pipeline stage of K), the metadata of the whole
// K extent stays in TMEM, and the pipeline stages hold activations only.
template <int NT, int KB>
struct PairResident {
  using T = PairTile<NT, KB>;
  static constexpr int kMaxStagesK = (kTmemCols - 2 * NT) / T::kMetaColsPerStage;   // TMEM left for metadata
  static constexpr int kFixed = T::kSaBytes + kPairEpiWarps * T::kStoreTile + 256 + 1024;
  // B pipeline stages that fit next to `slabs` resident A slabs (0 if fewer than 3)
  static int b_stages(int slabs) {
    const int room = 227 * 1024 - kFixed - slabs * T::kABytes;
    const int stages = room / T::kBBytes;
    return stages < 3 ? 0 : (stages > 8 ? 8 : stages);
  }
  static int smem_bytes(int slabs, int stages) { return slabs * T::kABytes + stages * T::kBBytes + kFixed; }
};

template <int NT, int KB, int MODE, bool RES = false, class Peers = NoPeers>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
sparse_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_e,
                        const __grid_constant__ CUtensorMap map_out, const KernelArgs args,
                        const __grid_constant__ Peers peers) {
  using T = PairTile<NT, KB>;
  constexpr bool INT32_OUT = MODE == kOutInt32, HAS_ADDEND = MODE == kOutBf16Addend;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int num_st = (args.num_kb + KB - 1) / KB;
  // pipeline depth and region offsets: compile-time in the streaming form, from the K extent in
  // the resident form (A slabs first, then the B stages, which also stage the metadata once)
  const int stages = RES ? args.res_stages : T::kStages;
  const int off_a = 0;
  const int off_b = RES ? num_st * T::kABytes : T::kOffB;
  const int off_e = RES ? off_b : T::kOffE;
  const int off_sa = RES ? off_b + stages * T::kBBytes : T::kOffSa;
  const int off_store = off_sa + T::kSaBytes;
  constexpr int kStoreBufs = RES ? 1 : T::kStoreBufs;
  const int off_bar = off_store + kStoreBufs * kPairEpiWarps * T::kStoreTile;
  constexpr int kBarStride = RES ? 8 : T::kStages;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + off_bar);
  uint64_t* bar_empty = bar_full + kBarStride;
  uint64_t* bar_acc_full = bar_empty + kBarStride;
  uint64_t* bar_acc_empty = bar_acc_full + T::kAccBufs;
  // streaming form: metadata of a stage is in TMEM (rank 0).  Resident form: [0] metadata of the
  // whole K extent is in TMEM (both CTAs), [1] resident operands have landed (rank 0)
  uint64_t* bar_meta = bar_acc_empty + T::kAccBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_meta + kBarStride);
  static_assert(!RES || T::kAccBufs == 2, "resident form assumes two accumulators");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_ch2 = (args.tiles_ch + 1) >> 1;            // tiles of 256 channels
  const int num_tiles = tiles_ch2 * args.tiles_tok;
  const bool meta_warp = !RES && args.meta_warp != 0;
  // Tile sequence of this cluster: pair, pair + num_pairs, ...; tile = token tile * tiles_ch2 +
  // channel tile.  The resident form is launched with a cluster count that is a multiple of
  // tiles_ch2, so every tile of a cluster has the same channel tile (tile % tiles_ch2).
  const int tile_first = pair, tile_step = num_pairs;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBarStride; ++s) {
      ptx::mbar_init(&bar_full[s], 1);
      ptx::mbar_init(&bar_empty[s], 1);
      ptx::mbar_init(&bar_meta[s], 1);
    }
    for (int b = 0; b < T::kAccBufs; ++b) {
      ptx::mbar_init(&bar_acc_full[b], 1);
      ptx::mbar_init(&bar_acc_empty[b], 2 * kPairEpiWarps);
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_e);
    if constexpr (MODE == kOutBf16Tma || MODE == kOutBf16GateAdd) ptx::prefetch_tensormap(&map_out);
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
    if (lane == 0) {
      uint32_t s = 0, phase = 0;       // pipeline stage and the parity of its current use
      bool ok = true;
      if constexpr (RES) {
        // the weights do not depend on the preceding kernel: fetch the resident operands first
        if (tile_first < num_tiles) {
          const int ch0 = (tile_first % tiles_ch2) * (2 * kTileCh) + static_cast<int>(rank) * kTileCh;
          if (rank == 0)
            ptx::mbar_arrive_expect_tx(&bar_meta[1], 2 * (num_st * T::kABytes + args.num_kb * T::kEBlock));
          for (int st = 0; st < num_st; ++st)
            ptx::tma_load_2d_pair(smem + off_a + st * T::kABytes, &map_a, &bar_meta[1], st * KB * (kBlockK / 2), ch0);
          for (int kb = 0; kb < args.num_kb; ++kb)
            ptx::tma_load_3d_pair(smem + off_e + kb * T::kEBlock, &map_e, &bar_meta[1], 0, kb, ch0 >> 5);
          // the metadata is staged where the first activation stages will live
          if (!ptx::mbar_wait(&bar_meta[0], 0)) ok = false;
        }
      }
      ptx::grid_dep_wait();           // q is written by the kernel launched just before this one
      for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step) {
        const int ch0 = (tile % tiles_ch2) * (2 * kTileCh) + static_cast<int>(rank) * kTileCh;
        const int tok0 = (tile / tiles_ch2) * NT + static_cast<int>(rank) * T::kHalf;
        for (int st = 0; st < num_st; ++st) {
          const int kb0 = st * KB;
          const int nkb = args.num_kb - kb0 < KB ? args.num_kb - kb0 : KB;
          if (!ptx::mbar_wait(&bar_empty[s], phase ^ 1u)) { ok = false; break; }
          if constexpr (RES) {
            if (rank == 0) ptx::mbar_arrive_expect_tx(&bar_full[s], 2 * nkb * T::kBBlock);
          } else {
            if (rank == 0)
              ptx::mbar_arrive_expect_tx(&bar_full[s], 2 * (T::kABytes + nkb * (T::kBBlock + T::kEBlock)));
            ptx::tma_load_2d_pair(smem + off_a + s * T::kABytes, &map_a, &bar_full[s], kb0 * (kBlockK / 2), ch0);
          }
          for (int h = 0; h < nkb; ++h) {
            ptx::tma_load_2d_pair(smem + off_b + s * T::kBBytes + h * T::kBBlock, &map_b, &bar_full[s],
                                  (kb0 + h) * kBlockK, tok0);
            if constexpr (!RES)
              ptx::tma_load_3d_pair(smem + off_e + s * T::kEBytes + h * T::kEBlock, &map_e, &bar_full[s], 0,
                                    kb0 + h, ch0 >> 5);
          }
          if (++s == static_cast<uint32_t>(stages)) { s = 0; phase ^= 1u; }
        }
      }
      if (!ok) atomicOr(args.status, kStatusProducerTimeout);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (rank 0 only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = (1u << 2) | (2u << 4) | (1u << 7) | (1u << 10) |
                                 (static_cast<uint32_t>(NT >> 3) << 17) |
                                 (static_cast<uint32_t>((2 * kTileCh) >> 4) << 24);
      constexpr uint32_t a_layout = KB == 2 ? 2u : 4u, a_sbo = KB == 2 ? 1024u : 512u;
      uint32_t s = 0, phase = 0, acc_it = 0;     // pipeline stage and the parity of its current use
      bool ok = true, ready = false;
      int release_stage = -1;        // stage whose MMAs are issued but whose barrier is not yet committed
      if constexpr (RES) {
        // once per cluster: metadata of the whole K extent from its staging area into TMEM
        if (tile_first < num_tiles) {
          if (!ptx::mbar_wait(&bar_meta[1], 0)) ok = false;
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
      for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step, ++acc_it) {
        const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
        if (!ptx::mbar_wait(&bar_acc_empty[buf], (acc_use & 1u) ^ 1u)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * NT;
        for (int st = 0; st < num_st; ++st) {
          const int kb0 = st * KB;
          const int nkb = args.num_kb - kb0 < KB ? args.num_kb - kb0 : KB;
          // with a metadata warp the stage is ready when its metadata copy has completed (which
          // implies that the operands have landed); without one this thread copies it itself
          uint64_t* bar_ready = meta_warp ? bar_meta : bar_full;
          if (!ready && !ptx::mbar_wait(&bar_ready[s], phase)) { ok = false; break; }
          ptx::tc_fence_after();
          // resident form: weights and metadata are indexed by the K position, not by the stage
          const uint32_t a_addr = ptx::smem_u32(smem + off_a + (RES ? st : static_cast<int>(s)) * T::kABytes);
          const uint32_t b_addr = ptx::smem_u32(smem + off_b + s * T::kBBytes);
          const uint32_t e_tmem = tmem_base + T::kMetaCol + (RES ? st : static_cast<int>(s)) * T::kMetaColsPerStage;
          if (!RES && !meta_warp) {
            const uint32_t e_addr = ptx::smem_u32(smem + off_e + s * T::kEBytes);
            if (KB == 2 && nkb == 2 && args.wide_cp) {
              // both metadata blocks of the stage in one instruction: block h is the h-th 16-byte
              // column of a 128 x 32-byte matrix whose columns lie kEBlock bytes apart
              ptx::tc_cp_128x256b_pair(e_tmem, smem_desc(e_addr, T::kEBlock, 128, 0));
            } else {
              for (int h = 0; h < nkb; ++h)
                ptx::tc_cp_128x128b_pair(e_tmem + 4 * h, smem_desc(e_addr + h * T::kEBlock, 128, 128, 0));
            }
          }
          const uint32_t s_next = s + 1 == static_cast<uint32_t>(stages) ? 0u : s + 1;
          const uint32_t phase_next = s_next == 0u ? phase ^ 1u : phase;
          for (int j = 0; j < 2 * nkb; ++j) {
            const uint64_t adesc = smem_desc(a_addr + j * 32, 16, a_sbo, a_layout);
            const uint64_t bdesc = smem_desc(b_addr + (j >> 1) * T::kBBlock + (j & 1) * 64, 16, 1024, 2);
            ptx::tc_mma_sp_i8_pair(d_tmem, adesc, bdesc, e_tmem + j * 2, idesc, (st | j) != 0 ? 1u : 0u);
            if (j == 0 && release_stage >= 0) {
              // the previous stage is handed back while this stage's first MMA keeps the pipe busy
              ptx::tc_commit_pair(&bar_empty[release_stage], 3);
              release_stage = -1;
            }
          }
          release_stage = static_cast<int>(s);
          // a look at the next stage's barrier once this stage's work is queued: it has usually
          // completed by now, and a successful look is far cheaper than a wait
          ready = mbar_peek(&bar_ready[s_next], phase_next);
          s = s_next;
          phase = phase_next;
        }
        if (release_stage >= 0) {
          ptx::tc_commit_pair(&bar_empty[release_stage], 3);
          release_stage = -1;
        }
        if (ok) ptx::tc_commit_pair(&bar_acc_full[buf], 3);
      }
      if (!ok) atomicOr(args.status, kStatusMmaTimeout);
    }
  } else if (warp == 2 + kPairEpiWarps) {
    // ------------------------------------------------------------------ metadata copier (rank 0 only)
    if (meta_warp && lane == 0 && rank == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step) {
        for (int st = 0; st < num_st; ++st) {
          const int kb0 = st * KB;
          const int nkb = args.num_kb - kb0 < KB ? args.num_kb - kb0 : KB;
          // the stage's previous metadata is no longer read once its MMAs have completed, which
          // the producer has already waited for before refilling the stage
          if (!ptx::mbar_wait(&bar_full[s], phase)) { ok = false; break; }
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
          ptx::tc_commit_pair(&bar_meta[s], 1);      // arrives (rank 0 only) when the copy has completed
          if (++s == static_cast<uint32_t>(stages)) { s = 0; phase ^= 1u; }
        }
      }
      if (!ok) atomicOr(args.status, kStatusMmaTimeout);
    }
  } else if constexpr (MODE == kOutBf16Tma || MODE == kOutBf16GateAdd || MODE == kOutBf16TmaPeers) {
    // ------------------------------------------------------------------ epilogue, TMA stores
    constexpr bool GATED = MODE == kOutBf16GateAdd;
    // The accumulator is channel-major in TMEM (lane = channel, column = token) and the output is
    // token-major.  tcgen05.ld in the 16x256b fragment layout hands each thread two adjacent
    // tokens of one channel per register pair, which is exactly what stmatrix.trans needs to
    // write 8 tokens x 8 channels blocks token-major: two values are converted with one packed
    // BF16 conversion and 32 of them stored with one stmatrix.x4.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    float* sa_s = reinterpret_cast<float*>(smem + off_sa) + (warp - 2) * NT;
    const int lane_ch = lane >> 2, tpair = (lane & 3) * 2;
    uint32_t acc_it = 0, store_it = 0;
    bool ok = true;
    constexpr int kSaRegs = (NT + 31) / 32;
    float sa_next[kSaRegs], sw_next[4], bias_next[4];
    auto prefetch = [&](int t) {
      const int pch = (t % tiles_ch2) * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32 + lane_ch;
      const int ptok0 = (t / tiles_ch2) * NT;
#pragma unroll
      for (int i = 0; i < kSaRegs; ++i) {
        const int tok = ptok0 + lane + 32 * i;
        sa_next[i] = (lane + 32 * i < NT && tok < args.m) ? __ldg(args.sa + tok) : 1.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {               // channels lane_ch + 8 i of the warp's 32
        const int c = pch + 8 * i;
        sw_next[i] = c < args.n ? __ldg(args.sw + c) : 1.f;
        bias_next[i] = (c < args.n && args.bias) ? __ldg(args.bias + c) : 0.f;
      }
    };
    ptx::grid_dep_wait();             // sa is written by the kernel launched just before this one
    if (tile_first < num_tiles) prefetch(tile_first);
    for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step, ++acc_it) {
      const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
      const int ch_w = (tile % tiles_ch2) * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32;
      const int tok0 = (tile / tiles_ch2) * NT;
      float sw[4], bias[4];
      __syncwarp();
#pragma unroll
      for (int i = 0; i < kSaRegs; ++i)
        if (lane + 32 * i < NT) sa_s[lane + 32 * i] = sa_next[i];
#pragma unroll
      for (int i = 0; i < 4; ++i) { sw[i] = sw_next[i]; bias[i] = bias_next[i]; }
      __syncwarp();
      if (tile + tile_step < num_tiles) prefetch(tile + tile_step);
      int chunks = (args.m - tok0 + 31) / 32;
      chunks = chunks < NT / 32 ? chunks : NT / 32;
      if (!ptx::mbar_wait(&bar_acc_full[buf], acc_use & 1u)) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * NT;
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_rank0(&bar_acc_empty[buf]);
      };
      auto load = [&](uint32_t (&f)[32], int c) {
        ptx::tc_ld_16x256b_x4(t_addr + c * 32, f);                       // channels 0..15 of the quadrant
        ptx::tc_ld_16x256b_x4(t_addr + (16u << 16) + c * 32, f + 16);    // channels 16..31
      };
      auto emit = [&](const uint32_t (&f)[32], int c) {
        uint8_t* stage = smem + off_store + ((warp - 2) * kStoreBufs + (store_it % kStoreBufs)) * T::kStoreTile;
        if (lane == 0) {
          if constexpr (kStoreBufs == 2) ptx::bulk_wait_read<1>(); else ptx::bulk_wait_read<0>();
        }
        __syncwarp();
        const float2* sa_c = reinterpret_cast<const float2*>(sa_s + c * 32 + tpair);
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
              const float2 s = sa_c[4 * g];                                  // tokens 8 g + tpair, + 1
              const uint32_t* r = f + 16 * h + 4 * g;
#pragma unroll
              for (int ab = 0; ab < 2; ++ab) {
                const float w = sw[2 * h + ab], b = bias[2 * h + ab];
                float y0 = __fmaf_rn(__int2float_rn(static_cast<int32_t>(r[2 * ab])), __fmul_rn(s.x, w), b);
                float y1 = __fmaf_rn(__int2float_rn(static_cast<int32_t>(r[2 * ab + 1])), __fmul_rn(s.y, w), b);
                if constexpr (GATED) {
                  y0 = __fmul_rn(gate[2 * h + ab], y0);
                  y1 = __fmul_rn(gate[2 * h + ab], y1);
                }
                const __nv_bfloat162 p = __floats2bfloat162_rn(y0, y1);     // low half = even token
                packed[2 * gi + ab] = *reinterpret_cast<const uint32_t*>(&p);
              }
            }
            const int tok = 8 * (2 * gp + (mi >> 1)) + (lane & 7);
            const int cg = 2 * h + (mi & 1);
            ptx::stmatrix_x4_trans(stage_addr + tok * 64 + ((cg ^ ((tok >> 1) & 3)) << 4),
                                   packed[0], packed[1], packed[2], packed[3]);
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          // rows >= m and channels >= n are clipped by the tensor map; a box that lies wholly
          // beyond the last channel is not issued at all
          if (ch_w < args.n) {
            if constexpr (GATED) {
              ptx::tma_reduce_add_2d(&map_out, stage, ch_w, tok0 + c * 32);
            } else if constexpr (MODE == kOutBf16TmaPeers) {
              // the same staged tile goes to this GPU's and every peer's gathered output
              for (int g = 0; g < args.peer_count; ++g) ptx::tma_store_2d(&peers.m[g], stage, ch_w, tok0 + c * 32);
            } else {
              ptx::tma_store_2d(&map_out, stage, ch_w, tok0 + c * 32);
            }
          }
          ptx::bulk_commit();
        }
        ++store_it;
      };
      const int mine = chunks > half ? (chunks - half + kPairSub - 1) / kPairSub : 0;
      if (mine == 0) {
        release();
      } else {
        uint32_t f0[32], f1[32];
        load(f0, half);
#pragma unroll 1
        for (int i = 0; i < mine; i += 2) {
          const int c = half + kPairSub * i;
          ptx::tc_wait_ld();
          if (i + 1 < mine) load(f1, c + kPairSub); else release();
          emit(f0, c);
          if (i + 1 < mine) {
            ptx::tc_wait_ld();
            if (i + 2 < mine) load(f0, c + 2 * kPairSub); else release();
            emit(f1, c + kPairSub);
          }
        }
      }
    }
    if (lane == 0) ptx::bulk_wait_all();
    __syncwarp();
    if (!ok && lane == 0) atomicOr(args.status, kStatusEpilogueTimeout);
  } else {
    // ------------------------------------------------------------------ epilogue, direct stores
    // (unaligned output, addend, INT32 dump): lane = channel, 32 token columns per tcgen05.ld
    const int quad = warp & 3;                    // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;             // which of the quadrant's warps: chunks half, half+kPairSub, ...
    float* sa_s = reinterpret_cast<float*>(smem + off_sa) + (warp - 2) * NT;
    uint32_t acc_it = 0;
    bool ok = true;
    // Scales of a tile are fetched one tile ahead into registers (the loads fly while the
    // previous tile is processed) and parked in shared memory when the tile starts.
    constexpr int kSaRegs = (NT + 31) / 32;
    float sa_next[kSaRegs], sw_next = 1.f, bias_next = 0.f;
    auto prefetch = [&](int t) {
      const int pch = (t % tiles_ch2) * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32 + lane;
      const int ptok0 = (t / tiles_ch2) * NT;
#pragma unroll
      for (int i = 0; i < kSaRegs; ++i) {
        const int tok = ptok0 + lane + 32 * i;
        sa_next[i] = (lane + 32 * i < NT && tok < args.m) ? __ldg(args.sa + tok) : 1.f;
      }
      sw_next = 1.f;
      bias_next = 0.f;
      if (pch < args.n) {
        sw_next = __ldg(args.sw + pch);
        if (args.bias) bias_next = __ldg(args.bias + pch);
      }
    };
    ptx::grid_dep_wait();
    if constexpr (!INT32_OUT) {
      if (tile_first < num_tiles) prefetch(tile_first);
    }
    for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step, ++acc_it) {
      const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
      const int ch = (tile % tiles_ch2) * (2 * kTileCh) + static_cast<int>(rank) * kTileCh + quad * 32 + lane;
      const int tok0 = (tile / tiles_ch2) * NT;
      const bool ch_ok = ch < args.n;
      float sw = 1.f, bias = 0.f;
      if constexpr (!INT32_OUT) {
        __syncwarp();
#pragma unroll
        for (int i = 0; i < kSaRegs; ++i)
          if (lane + 32 * i < NT) sa_s[lane + 32 * i] = sa_next[i];
        sw = sw_next;
        bias = bias_next;
        __syncwarp();
        if (tile + tile_step < num_tiles) prefetch(tile + tile_step);
      }
      int chunks = (args.m - tok0 + 31) / 32;
      chunks = chunks < NT / 32 ? chunks : NT / 32;
      if (!ptx::mbar_wait(&bar_acc_full[buf], acc_use & 1u)) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * NT;
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_rank0(&bar_acc_empty[buf]);
      };
      uint32_t r0[32], r1[32];
      auto emit = [&](const uint32_t (&r)[32], int c) {
        store_chunk<INT32_OUT, HAS_ADDEND>(r, args, sa_s + c * 32, tok0 + c * 32, ch, ch_ok, sw, bias);
      };
      const int mine = chunks > half ? (chunks - half + kPairSub - 1) / kPairSub : 0;
      if (mine == 0) {
        release();
      } else {
        ptx::tc_ld_32x32b_x32(t_addr + half * 32, r0);
#pragma unroll 1
        for (int i = 0; i < mine; i += 2) {
          const int c = half + kPairSub * i;
          ptx::tc_wait_ld();
          if (i + 1 < mine) ptx::tc_ld_32x32b_x32(t_addr + (c + kPairSub) * 32, r1); else release();
          emit(r0, c);
          if (i + 1 < mine) {
            ptx::tc_wait_ld();
            if (i + 2 < mine) ptx::tc_ld_32x32b_x32(t_addr + (c + 2 * kPairSub) * 32, r0); else release();
            emit(r1, c + kPairSub);
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
