// 2:4 sparse INT8 GEMM for sm_100a: tcgen05.mma.sp (kind::i8) with TMA-fed shared-memory
// stages, INT32 accumulators in tensor memory and a fused dequant / bias / addend / BF16 epilogue.
//
//   acc[ch, tok] = sum_c  W_lifted[ch, c] * q[tok, c]          (exact int32)
//   out[tok, ch] = bf16( fma(float(acc), sa[tok]*sw[ch], bias[ch]) [+ float(addend[tok,ch])] )
//
// The 2:4-compressed weights are the sparse A operand (UMMA M = 128 output channels per SM),
// the quantised activations are B (UMMA N = token tile), so the accumulator lanes are channels
// and its columns are tokens, as in the reference (csrc/dualscale_sm80.cu:189-204).
//
// There is one kernel, sparse_gemm_pair_kernel (ss_gemm_pair.cuh): persistent clusters of two CTAs
// (cta_group::2), warp-specialised into a TMA producer, an MMA issuer, a metadata copier and eight
// epilogue warps per CTA, with two accumulators in TMEM so that the epilogue of one tile overlaps
// the main loop of the next.  This file holds what the kernel needs around it: argument block,
// descriptor helpers, the direct-store epilogue body, tile choice, tensor maps and the launch.
// Every mbarrier wait is bounded; a wait that runs out records a code in the device status word
// and the CTA winds down.
#include "ss_common.cuh"
#include <cuda_bf16.h>
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace ss {
namespace {

constexpr int kTileCh = 128;                     // UMMA M per SM
constexpr int kBlockK = 128;                     // lifted columns per metadata / B block
constexpr int kTmemCols = 512;

struct KernelArgs {
  const float* sa;
  const float* sw;
  const float* bias;
  const __nv_bfloat16* addend;
  long long addend_stride;
  void* out;
  long long out_stride;
  int m, n;
  int tiles_ch, tiles_tok, num_kb;
  uint32_t* status;
  int wide_cp;          // CTA-pair kernel: copy a stage's two metadata blocks with one tcgen05.cp
  int meta_warp;        // CTA-pair kernel: a dedicated warp issues the metadata copies
  const __nv_bfloat16* gate;   // gated accumulation: BF16 [batches, n], rows gate_stride apart
  long long gate_stride;
  int rows_per_batch;
  int res_stages;       // weights-resident form: activation pipeline stages
  int peer_count;       // tensor-parallel form: number of destination tensor maps
  unsigned long long wait_ns;      // limit of every mbarrier wait
  int debug;                       // diagnostics: bit 0 no MMAs, 1 no epilogue work, 2 no TMA stores, 3 TMEM loads only
  unsigned long long* probe;       // diagnostics: cluster 0 writes {cycles of its tile loop, stages}
  int out_evict_first;             // TMA stores of the output carry the L2 evict_first hint
  int32_t* split_sum;              // split schedule: the clusters' slabs for pieces of shared tiles
  int* split_ticket;               // split schedule: arrivals per epilogue warp of a shared tile (zero between launches)
};

__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= 1ull << 46;                                   // descriptor version of this architecture
  d |= static_cast<uint64_t>(layout_type) << 61;     // 0 none, 2 128B, 4 64B swizzle
  return d;
}

// Dequantise one 32-token chunk held in registers (lane = channel) and store it.  sa_lane is the
// scale of token tok_base + lane; the lanes hand each other the scale of the token being written.
template <bool INT32_OUT, bool HAS_ADDEND>
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], const KernelArgs& args,
                                            float sa_lane, int tok_base, int tok_end, int ch,
                                            bool ch_ok, float sw, float bias) {
  if constexpr (INT32_OUT) {
    int32_t* out = static_cast<int32_t*>(args.out);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (ch_ok && tok_base + j < tok_end)
        out[static_cast<long long>(tok_base + j) * args.out_stride + ch] = static_cast<int32_t>(r[j]);
  } else {
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(args.out);
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j4 * 4 + jj, tok = tok_base + j;
        const float sa_tok = __shfl_sync(0xffffffffu, sa_lane, j);
        float y = __fmaf_rn(__int2float_rn(static_cast<int32_t>(r[j])), __fmul_rn(sa_tok, sw), bias);
        if (ch_ok && tok < tok_end) {
          if constexpr (HAS_ADDEND)
            y = __fadd_rn(y, __bfloat162float(args.addend[static_cast<long long>(tok) * args.addend_stride + ch]));
          out[static_cast<long long>(tok) * args.out_stride + ch] = __float2bfloat16_rn(y);
        }
      }
    }
  }
}

#include "ss_gemm_pair.cuh"

// ---- host side -----------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
    uint64_t h = 1469598103934665603ull;                  // FNV-1a over the whole (zero-padded) key
    for (size_t i = 0; i < sizeof(MapKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
    return static_cast<size_t>(h);
  }
};
struct MapKeyEq {
  bool operator()(const MapKey& a, const MapKey& b) const { return std::memcmp(&a, &b, sizeof(MapKey)) == 0; }
};
constexpr size_t kMapCacheLimit = 8192;   // descriptors kept; the cache starts over beyond this

// kernel variants: token tile x output mode x resident form
constexpr int kTileCount = 5, kModeCount = 7;
struct DeviceInfo {
  int sms = 0;
  std::atomic<bool> configured[kTileCount][kModeCount][2];
  // split schedule: two accumulator slabs per cluster and one ticket per epilogue warp (tickets zero
  // between launches).  Launches on different streams may overlap, so each stream that launches the
  // split schedule gets an area of its own out of a pool of kSplitAreas, allocated as a whole by the
  // first such launch outside a stream capture (handing an area to a stream needs no CUDA call, so a
  // capturing stream can still get one).  An area whose launches were all eager and have completed
  // (an event recorded after each) goes to the next stream that asks; one used inside a capture stays
  // with its stream, since the graph may be replayed at any time.  Streams that find no area, and
  // captures before the pool exists, keep whole tiles.
  static constexpr int kSplitAreas = 4;
  struct SplitArea { cudaStream_t stream; int32_t* sum; int* ticket; cudaEvent_t done; bool pinned; bool used; int claims; };
  std::mutex split_mu;
  SplitArea split_area[kSplitAreas] = {};
  int split_areas = 0;            // areas handed to streams
  void* split_pool = nullptr;
  size_t split_bytes = 0;         // bytes of one area
  DeviceInfo() { for (auto& a : configured) for (auto& b : a) for (auto& c : b) c.store(false); }
};
DeviceInfo* device_info() {
  static std::mutex mu;
  static std::unordered_map<int, DeviceInfo*> table;      // entries live for the process
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  auto it = table.find(dev);
  if (it != table.end()) return it->second;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return nullptr;
  DeviceInfo* d = new DeviceInfo();
  d->sms = sms;
  table[dev] = d;
  return d;
}

// Token tile of a launch (256 channels x NT tokens per cluster): the candidate with the smallest
// rounds x cost-per-tile; ties go to the smaller tile.  Cost of one tile in cycles = blocks of 128
// lifted columns x per-block cost + per-tile cost, both fitted per token tile (relative least
// squares) to GEMM times measured by CUDA-graph replay over 23 shapes of the benchmark
// configurations (K' 1152 .. 18432, M 256 .. 16384).  The per-tile part is the pipeline fill, the
// epilogue tail and the barrier round trips; 256 has a single accumulator, so its epilogue is
// exposed.  Over those shapes the model's choice costs 0.4 % more than the best tile per shape.
std::atomic<long long> g_split_launches{0};

// The split schedule's area of `stream`, handed out now if `create` and one is left (the pool is
// allocated here too, unless `stream` is capturing); nullptr if there is none.
DeviceInfo::SplitArea* split_workspace(DeviceInfo* dev, cudaStream_t stream, bool create) {
  std::lock_guard<std::mutex> lock(dev->split_mu);
  // `create` is the call of a launch that is about to use the area: it holds a claim on it until
  // the launch has been issued (released in launch_gemm), so that no other thread's launch takes it
  for (int i = 0; i < dev->split_areas; ++i)
    if (dev->split_area[i].stream == stream) {
      if (create) ++dev->split_area[i].claims;
      return &dev->split_area[i];
    }
  if (!create) return nullptr;
  if (dev->split_areas == DeviceInfo::kSplitAreas) {
    for (DeviceInfo::SplitArea& area : dev->split_area) {
      if (area.pinned || area.claims > 0 || (area.used && cudaEventQuery(area.done) != cudaSuccess)) continue;
      area.stream = stream;          // its launches have completed: tickets are zero again
      area.used = false;
      area.claims = 1;
      return &area;
    }
    cudaGetLastError();
    return nullptr;
  }
  const size_t clusters = static_cast<size_t>(dev->sms / 2);
  const size_t sum_bytes = clusters * 2 * static_cast<size_t>(kSplitClusterWords) * sizeof(int32_t);   // two slabs per cluster
  const size_t ticket_bytes = (clusters * 2 * kPairEpiWarps * sizeof(int) + 255) / 256 * 256;
  if (!dev->split_pool) {
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      return nullptr;
    }
    const size_t total = (sum_bytes + ticket_bytes) * DeviceInfo::kSplitAreas;
    void* p = nullptr;
    if (cudaMalloc(&p, total) != cudaSuccess || cudaMemset(p, 0, total) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
      cudaGetLastError();
      if (p) cudaFree(p);
      return nullptr;
    }
    for (DeviceInfo::SplitArea& area : dev->split_area) {
      if (cudaEventCreateWithFlags(&area.done, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return nullptr;
      }
    }
    dev->split_pool = p;
    dev->split_bytes = sum_bytes + ticket_bytes;
  }
  DeviceInfo::SplitArea& area = dev->split_area[dev->split_areas];
  char* base = static_cast<char*>(dev->split_pool) + dev->split_bytes * dev->split_areas;
  area.stream = stream;
  area.sum = reinterpret_cast<int32_t*>(base);
  area.ticket = reinterpret_cast<int*>(base + sum_bytes);
  area.pinned = false;
  area.used = false;
  area.claims = 1;
  ++dev->split_areas;
  return &area;
}

constexpr int kTiles[kTileCount] = {128, 192, 224, 240, 256};
constexpr double kPerBlock[kTileCount] = {351.0, 415.0, 414.0, 425.0, 448.0};
constexpr double kPerTile[kTileCount] = {2477.0, 2813.0, 4107.0, 3925.0, 5799.0};

// Split schedule (see Walk in ss_gemm_pair.cuh): the clusters share the tiles x stages evenly, so a
// launch costs tiles / clusters (not rounded up) tile costs, plus what the shared tiles cost: every
// cluster stores one accumulator to global memory at the start of its range and fetches one at the
// end, where nothing hides it, and the clusters no longer walk K in step (measured over 20 shapes:
// 5-6 us, of which the last piece's fetch and epilogue are about 2 us).  It therefore pays only when
// a whole-tile launch would idle most clusters through a long last round, e.g. 2048 x 9728 -> 2432
// (4:6): 100 tiles of 76 stages on 74 clusters, 42.7 -> 38.3 us.
constexpr double kSplitExtra = 11000.0;

struct TilePick { int nt; double cost; };
TilePick pick_pair_token_tile(int64_t m, int64_t pn, int64_t pk, int sms, bool whole_chunks_only, bool split = false) {
  const int forced = options().token_tile;
  const int64_t tiles_ch2 = (pn + 2 * kTileCh - 1) / (2 * kTileCh);
  const double num_kb = static_cast<double>(pk / kBlockK);
  const int64_t pairs = sms / 2 > 0 ? sms / 2 : 1;
  TilePick best{224, 0};
  for (int i = 0; i < kTileCount; ++i) {
    const int nt = kTiles[i];
    if (whole_chunks_only && nt % 32) continue;
    if (forced && forced != nt) continue;
    const int64_t tiles = tiles_ch2 * ((m + nt - 1) / nt);
    const double per_tile = num_kb * kPerBlock[i] + kPerTile[i];
    double cost;
    if (split) {
      // with fewer tiles than clusters a tile is shared by many and its last piece adds up many
      // slabs: measured slower than the whole-tile schedule throughout, unless forced
      if (tiles < pairs && options().split != 1) continue;
      const double rounds = static_cast<double>(tiles) / static_cast<double>(pairs);
      cost = (rounds < 1.0 ? num_kb * kPerBlock[i] * rounds + kPerTile[i] : rounds * per_tile) + kSplitExtra;
    } else {
      cost = static_cast<double>((tiles + pairs - 1) / pairs) * per_tile;
    }
    if (best.cost == 0 || cost < best.cost * 0.999) best = {nt, cost};
  }
  if (best.cost == 0 && !split) {          // a forced tile the form excludes (the half chunk of 240): as if none were forced
    for (int i = 0; i < kTileCount; ++i) {
      const int nt = kTiles[i];
      if (whole_chunks_only && nt % 32) continue;
      const int64_t tiles = tiles_ch2 * ((m + nt - 1) / nt);
      const double cost = static_cast<double>((tiles + pairs - 1) / pairs) * (num_kb * kPerBlock[i] + kPerTile[i]);
      if (best.cost == 0 || cost < best.cost * 0.999) best = {nt, cost};
    }
  }
  return best;
}

// ---- launcher ----------------------------------------------------------------------------------
// RES: weights-resident form (see PairResident); res_stages = its activation pipeline depth.
template <int NT, int KB, int MODE, bool RES = false>
int launch_pair_t(const GemmArgs& a, DeviceInfo* dev, int tile_index, cudaStream_t stream, int res_stages = 0) {
  using T = PairTile<NT, KB>;
  using Peers = std::conditional_t<MODE == kOutBf16TmaPeers, PeerMaps, NoPeers>;
  auto kernel = sparse_gemm_pair_kernel<NT, KB, MODE, RES, Peers>;
  std::atomic<bool>& configured = dev->configured[tile_index][MODE][RES];
  if (!configured.load(std::memory_order_acquire)) {
    // idempotent: two host threads that race here both set the same value
    SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 RES ? 227 * 1024 : T::kSmemBytes));
    configured.store(true, std::memory_order_release);
  }
  const Options& opt = options();
  CUtensorMap map_a, map_b, map_e, map_out, map_out_tail;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.pk / 2), static_cast<cuuint64_t>(a.pn)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.pk / 2)};
    const cuuint32_t box[2] = {kBlockK / 2 * KB, kTileCh};
    int rc = encode_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.packed, dims, strides, box,
                        KB == 2 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  const cuuint64_t kblocks = static_cast<cuuint64_t>(a.pk / kBlockK);
  {
    // q[pm, pk] seen as [block of 128 columns][token][128 bytes]: one box = this CTA's half of the
    // token rows for the KB blocks of a stage, block after block in shared memory
    const cuuint64_t dims[3] = {kBlockK, static_cast<cuuint64_t>(a.pm), kblocks};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(a.pk), kBlockK};
    const cuuint32_t box[3] = {kBlockK, T::kHalf, KB};
    int rc = encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    // metadata seen as [block of 128 columns][group of 32 rows][128 words]: one box = the four row
    // groups of this CTA's 128 channels for the KB blocks of a stage, 2 KB per block, block after block
    const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(a.pn / 32), kblocks};
    const cuuint64_t strides[2] = {kblocks * 512, 512};
    const cuuint32_t box[3] = {128, 4, KB};
    int rc = encode_map(&map_e, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, a.meta, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  KernelArgs k;
  k.sa = a.sa; k.sw = a.sw; k.bias = a.bias;
  k.addend = static_cast<const __nv_bfloat16*>(a.addend);
  k.addend_stride = a.addend_stride;
  k.out = a.out; k.out_stride = a.out_stride;
  k.m = static_cast<int>(a.m); k.n = static_cast<int>(a.n);
  k.tiles_ch = static_cast<int>((a.pn + kTileCh - 1) / kTileCh);
  k.tiles_tok = static_cast<int>((a.m + NT - 1) / NT);
  k.num_kb = static_cast<int>(a.pk / kBlockK);
  k.status = device_status_ptr();
  SS_REQUIRE(k.status, SS_E_CUDA, "device status word unavailable");
  k.gate = static_cast<const __nv_bfloat16*>(a.gate);
  k.gate_stride = a.gate_stride;
  k.rows_per_batch = static_cast<int>(a.rows_per_batch);
  k.wide_cp = opt.wide_cp;
  k.meta_warp = opt.meta_warp >= 0 ? opt.meta_warp : (T::kStages >= 4 ? 1 : 0);
  k.res_stages = res_stages;
  k.peer_count = 0;
  k.wait_ns = a.wait_ns ? a.wait_ns : opt.wait_ns;
  k.debug = a.debug;
  k.probe = a.probe;
  // an output of at least half the L2 (126 MB) leaves as evict_first: measured -1.3 % on
  // 16384 x 3072 -> 12288 (403 MB out), -1 % on 4096 x 3072 -> 12288 (101 MB), nothing below; a
  // smaller output is left for the kernel that consumes it
  k.out_evict_first = 2 * a.m * a.n >= (63ll << 20) ? 1 : 0;
  k.split_sum = nullptr;
  k.split_ticket = nullptr;
  DeviceInfo::SplitArea* split_area = nullptr;
  if constexpr (MODE == kOutBf16TmaSplit) {
    split_area = split_workspace(dev, stream, false);
    if (split_area) {
      k.split_sum = split_area->sum;
      k.split_ticket = split_area->ticket;
    }
    g_split_launches.fetch_add(1, std::memory_order_relaxed);
  }
  const int64_t tiles_ch2 = (k.tiles_ch + 1) / 2;
  const int64_t tiles = tiles_ch2 * k.tiles_tok;
  const int64_t pairs = dev->sms / 2;
  unsigned grid = 2u * static_cast<unsigned>(tiles < pairs ? tiles : pairs);
  if constexpr (MODE == kOutBf16TmaSplit) {
    // every cluster takes an equal share of the tiles x stages
    SS_REQUIRE(k.split_sum && k.split_ticket, SS_E_ARG, "gemm: the split schedule has no tile-sum area");
    const int64_t units = tiles * ((k.num_kb + KB - 1) / KB);
    grid = 2u * static_cast<unsigned>(units < pairs ? units : pairs);
  }
  int smem_bytes = T::kSmemBytes;
  if constexpr (RES) {
    // a whole number of clusters per channel tile, so that a cluster never changes its weights
    int64_t group = pairs / tiles_ch2;
    if (group > k.tiles_tok) group = k.tiles_tok;
    SS_REQUIRE(group >= 1 && res_stages >= 3, SS_E_ARG, "gemm: resident form not applicable");
    grid = 2u * static_cast<unsigned>(group * tiles_ch2);
    smem_bytes = PairResident<NT, KB>::smem_bytes((k.num_kb + KB - 1) / KB);
  }
  map_out = map_a;         // unused by the direct-store epilogues
  map_out_tail = map_a;
  if constexpr (MODE == kOutBf16Tma || MODE == kOutBf16GateAdd || MODE == kOutBf16TmaSplit) {
    // out[m, n] BF16, row pitch out_stride: one 32-channel x 32-token box per epilogue warp and chunk;
    // the epilogue writes its 64-byte rows with the 16-byte pieces XOR-swizzled (bank-conflict-free stmatrix)
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.out_stride) * 2};
    const cuuint32_t box[2] = {32, 32};
    int rc = encode_map(&map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    if constexpr (T::kHalfTail) {
      const cuuint32_t half_box[2] = {32, 16};
      rc = encode_map(&map_out_tail, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.out, dims, strides, half_box,
                      CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc) return rc;
    }
  }
  Peers peers{};
  if constexpr (MODE == kOutBf16TmaPeers) {
    SS_REQUIRE(a.peer_count >= 1 && a.peer_count <= kMaxPeers, SS_E_ARG, "gemm: 1..%d destinations", kMaxPeers);
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.out_stride) * 2};
    const cuuint32_t box[2] = {32, 32};
    for (int g = 0; g < a.peer_count; ++g) {
      SS_REQUIRE(a.peer_out[g] && (reinterpret_cast<uintptr_t>(a.peer_out[g]) & 15) == 0, SS_E_ARG,
                 "gemm: destination %d must be a 16-byte aligned pointer", g);
      int rc = encode_map(&peers.m[g], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.peer_out[g], dims, strides,
                          box, CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc) return rc;
    }
    k.peer_count = a.peer_count;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.overlap_prologue && opt.pdl ? 1 : 0;
  SS_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_e, map_out, map_out_tail, k, peers));
  SS_CUDA(cudaGetLastError());
  if (split_area) {
    // when this area may go to another stream: after this launch if it is an eager one, never if it
    // is part of a capture (the graph may be replayed at any time)
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    SS_CUDA(cudaStreamIsCapturing(stream, &capture));
    std::lock_guard<std::mutex> lock(dev->split_mu);
    if (capture != cudaStreamCaptureStatusNone) {
      split_area->pinned = true;
    } else {
      SS_CUDA(cudaEventRecord(split_area->done, stream));
      split_area->used = true;
    }
  }
  return SS_OK;
}

// Weights-resident form: applicable when the K extent's metadata fits the TMEM columns left beside
// two accumulators and there are no more channel tiles than clusters; worth using (measured) only
// when at least four activation stages fit next to the weights (lifted K up to about 1300: with
// three the pipeline is too shallow, 6:8 at K = 1152 ran 30 % slower) and a cluster sees at least
// four token tiles (the weights are fetched before the first MMA; with two tiles that start-up
// costs more than the re-use saves).  Returns the activation pipeline depth, 0 if not applicable.
template <int NT>
int resident_stages(const GemmArgs& a, int sms) {
  using R = PairResident<NT, 2>;
  const int64_t num_kb = a.pk / kBlockK, slabs = (num_kb + 1) / 2;
  const int64_t tiles_ch2 = (a.pn + 2 * kTileCh - 1) / (2 * kTileCh), tiles_tok = (a.m + NT - 1) / NT;
  const int64_t pairs = sms / 2;
  if (slabs > R::kMaxStagesK || tiles_ch2 > pairs) return 0;
  const int stages = R::b_stages(static_cast<int>(slabs));
  if (stages < 4 || num_kb * R::T::kEBlock > static_cast<int64_t>(stages) * R::T::kBBytes) return 0;
  const int64_t group = pairs / tiles_ch2;
  if (tiles_tok < 4 * group) return 0;
  return stages;
}

// TMA stores need a 16-byte aligned base and row pitch, and a channel count that is a multiple of 8:
// a tiled store that crosses the tensor's channel extent is cut at the next 16-byte boundary, not at
// the extent, so with n % 8 != 0 and a row pitch wider than n it would write up to 7 zero-padded
// channels into the columns beside the output
bool tma_store_ok(const GemmArgs& a) {
  return (reinterpret_cast<uintptr_t>(a.out) & 15) == 0 && a.out_stride % 8 == 0 && a.n % 8 == 0;
}

template <int NT, int KB>
int launch_pair_nt(const GemmArgs& a, DeviceInfo* dev, int tile_index, cudaStream_t stream, int res_stages = 0, bool split = false) {
  if (split) return launch_pair_t<NT, KB, kOutBf16TmaSplit>(a, dev, tile_index, stream);
  if (a.int32_out) return launch_pair_t<NT, KB, kOutInt32>(a, dev, tile_index, stream);
  if (a.addend) return launch_pair_t<NT, KB, kOutBf16Addend>(a, dev, tile_index, stream);
  const bool aligned = tma_store_ok(a);
  if constexpr (KB == 2 && (NT == 192 || NT == 224)) {
    if (res_stages > 0 && aligned) {
      if (a.gate) return launch_pair_t<NT, KB, kOutBf16GateAdd, true>(a, dev, tile_index, stream, res_stages);
      return launch_pair_t<NT, KB, kOutBf16Tma, true>(a, dev, tile_index, stream, res_stages);
    }
  }
  if (a.gate) {
    SS_REQUIRE(aligned, SS_E_ARG, "gated accumulation needs a 16-byte aligned output and row pitch and n % 8 == 0");
    return launch_pair_t<NT, KB, kOutBf16GateAdd>(a, dev, tile_index, stream);
  }
  if constexpr (NT % 32 == 0) {
    if (a.peer_count > 0) {
      SS_REQUIRE(a.out_stride % 8 == 0 && a.n % 8 == 0, SS_E_ARG,
                 "tensor-parallel stores need a shard width and a row pitch that are multiples of 8");
      return launch_pair_t<NT, KB, kOutBf16TmaPeers>(a, dev, tile_index, stream);
    }
  }
  if (aligned && options().store == 1) return launch_pair_t<NT, KB, kOutBf16Tma>(a, dev, tile_index, stream);
  return launch_pair_t<NT, KB, kOutBf16>(a, dev, tile_index, stream);
}

int check_args(const GemmArgs& a) {
  SS_REQUIRE(a.q && a.packed && a.meta && (a.out || a.peer_count > 0), SS_E_ARG, "gemm: null pointer");
  SS_REQUIRE(a.peer_count == 0 || (!a.int32_out && !a.addend && !a.gate), SS_E_ARG,
             "gemm: the tensor-parallel form excludes addend, gate and the INT32 dump");
  SS_REQUIRE(a.int32_out || (a.sa && a.sw), SS_E_ARG, "gemm: scales required");
  SS_REQUIRE(a.pk > 0 && a.pk % 128 == 0 && a.pm > 0 && a.pm % 32 == 0 && a.pn > 0 && a.pn % 32 == 0,
             SS_E_ARG, "gemm: padding mismatch (pm=%lld pn=%lld pk=%lld)", (long long)a.pm, (long long)a.pn, (long long)a.pk);
  SS_REQUIRE(a.pk <= 131008, SS_E_ARG, "gemm: INT32 worst-case bound exceeded (pk=%lld)", (long long)a.pk);
  SS_REQUIRE(a.m > 0 && a.m <= a.pm && a.n > 0 && a.n <= a.pn, SS_E_ARG,
             "gemm: original dimensions exceed the padded ones (m=%lld n=%lld)", (long long)a.m, (long long)a.n);
  SS_REQUIRE(a.pm < (1ll << 31) && a.pn < (1ll << 31), SS_E_ARG, "gemm: dimension too large");
  SS_REQUIRE(a.out_stride >= a.n, SS_E_ARG, "gemm: output row stride smaller than n");
  SS_REQUIRE((reinterpret_cast<uintptr_t>(a.q) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.packed) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(a.meta) & 15) == 0,
             SS_E_ARG, "gemm: q, packed and metadata must be 16-byte aligned");
  SS_REQUIRE(a.int32_out || (reinterpret_cast<uintptr_t>(a.sa) & 15) == 0, SS_E_ARG,
             "gemm: token scales must be 16-byte aligned");
  SS_REQUIRE(!a.addend || a.addend_stride >= a.n, SS_E_ARG, "gemm: addend row stride smaller than n");
  if (a.gate) {
    SS_REQUIRE(!a.int32_out && !a.addend, SS_E_ARG, "gemm: gated accumulation excludes the addend and the INT32 dump");
    SS_REQUIRE(a.rows_per_batch > 0 && a.rows_per_batch % 32 == 0 && a.rows_per_batch < (1ll << 31), SS_E_ARG,
               "gemm: gated accumulation needs rows_per_batch to be a positive multiple of 32 (got %lld)",
               (long long)a.rows_per_batch);
    SS_REQUIRE(a.gate_stride >= a.n, SS_E_ARG, "gemm: gate row stride smaller than n");
  }
  return SS_OK;
}

// The tile and form launch_gemm uses for a problem: token tile, resident pipeline depth (0 = the
// streaming form).
struct Choice { int nt; int res_stages; bool split; };
Choice choose(const GemmArgs& a, int sms, bool split_allowed) {
  const Options& opt = options();
  if (opt.resident && !a.int32_out && !a.addend && a.peer_count == 0 && opt.token_tile == 0 && tma_store_ok(a)) {
    // prefer the token tile that needs fewer rounds of the clusters that share a channel tile
    const int s224 = resident_stages<224>(a, sms), s192 = resident_stages<192>(a, sms);
    const int64_t tiles_ch2 = (a.pn + 2 * kTileCh - 1) / (2 * kTileCh), group = (sms / 2) / (tiles_ch2 ? tiles_ch2 : 1);
    auto rounds = [&](int nt) { const int64_t t = (a.m + nt - 1) / nt; return (t + group - 1) / group; };
    if (s224 && (!s192 || rounds(224) * 224 <= rounds(192) * 192)) return {224, s224, false};
    if (s192) return {192, s192, false};
  }
  // the half chunk of the 240-token tile exists in the TMA-store epilogues only
  const bool whole_chunks_only = a.peer_count > 0;
  const TilePick whole = pick_pair_token_tile(a.m, a.pn, a.pk, sms, whole_chunks_only);
  // the split schedule: plain aligned BF16 output only, at least two stages per tile, and worth its
  // extra trip through global memory by the cost model (or forced)
  if (split_allowed && opt.split != 0 && a.allow_split && opt.store == 1 && !a.int32_out && !a.addend && !a.gate &&
      a.peer_count == 0 && tma_store_ok(a) && a.pk / kBlockK >= 4) {
    const TilePick shared = pick_pair_token_tile(a.m, a.pn, a.pk, sms, false, true);
    if (shared.cost > 0 && (opt.split == 1 || shared.cost < 0.93 * whole.cost)) return {shared.nt, 0, true};
  }
  return {whole.nt, 0, false};
}

}  // namespace

Options& options() {
  static Options* opt = [] {
    Options* o = new Options();
    auto read = [](const char* name, int fallback) {
      const char* env = std::getenv(name);
      return env ? std::atoi(env) : fallback;
    };
    o->token_tile = read("SS_TOKEN_TILE", 0);
    o->wide_cp = read("SS_WIDE_CP", 1);
    o->meta_warp = read("SS_META_WARP", -1);
    o->store = read("SS_STORE", 1);
    o->resident = read("SS_RESIDENT", 1);
    o->pdl = read("SS_PDL", 1);
    o->split = read("SS_SPLIT", -1);
    if (const char* env = std::getenv("SS_WAIT_NS")) {
      const long long v = std::atoll(env);
      if (v > 0) o->wait_ns = static_cast<unsigned long long>(v);
    }
    return o;
  }();
  return *opt;
}

int encode_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base,
               const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
               CUtensorMapSwizzle swizzle) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash, MapKeyEq> cache;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.type = static_cast<int>(type);
  key.rank = rank;
  key.swizzle = static_cast<int>(swizzle);
  for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return SS_OK;
    }
  }
  EncodeFn fn = encode_fn();
  SS_REQUIRE(fn, SS_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint32_t ones[3] = {1, 1, 1};
  CUresult r = fn(map, type, rank, const_cast<void*>(base), dims, strides, box, ones,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SS_REQUIRE(r == CUDA_SUCCESS, SS_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() >= kMapCacheLimit) cache.clear();
  cache.emplace(key, *map);
  return SS_OK;
}

int launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (int rc = check_args(a)) return rc;
  DeviceInfo* dev = device_info();
  SS_REQUIRE(dev, SS_E_CUDA, "gemm: no current CUDA device");
  Choice c = choose(a, dev->sms, true);
  // the tile-sum area is made on the first launch that wants it; a launch that cannot have it (a
  // stream capture before any such launch, no memory) takes the whole-tile schedule
  DeviceInfo::SplitArea* area = c.split ? split_workspace(dev, stream, true) : nullptr;
  if (c.split && !area) c = choose(a, dev->sms, false);
  int rc;
  switch (c.nt) {
    case 128: rc = launch_pair_nt<128, 2>(a, dev, 0, stream, 0, c.split); break;
    case 192: rc = launch_pair_nt<192, 2>(a, dev, 1, stream, c.res_stages, c.split); break;
    case 224: rc = launch_pair_nt<224, 2>(a, dev, 2, stream, c.res_stages, c.split); break;
    case 240: rc = launch_pair_nt<240, 2>(a, dev, 3, stream, 0, c.split); break;
    default:  rc = launch_pair_nt<256, 2>(a, dev, 4, stream, 0, c.split); break;
  }
  if (area) {
    std::lock_guard<std::mutex> lock(dev->split_mu);
    --area->claims;
  }
  return rc;
}

long long split_launch_count() { return g_split_launches.load(std::memory_order_relaxed); }

int reset_split_workspace() {
  DeviceInfo* dev = device_info();
  SS_REQUIRE(dev, SS_E_CUDA, "no current CUDA device");
  std::lock_guard<std::mutex> lock(dev->split_mu);
  if (!dev->split_pool) return SS_OK;
  SS_CUDA(cudaMemset(dev->split_pool, 0, dev->split_bytes * DeviceInfo::kSplitAreas));
  SS_CUDA(cudaDeviceSynchronize());
  return SS_OK;
}

template <int NT, int KB>
static int pair_resources_t(GemmResources* r, int res_stages, int slabs, bool split = false) {
  using T = PairTile<NT, KB>;
  cudaFuncAttributes attr;
  int smem = T::kSmemBytes, stages = T::kStages;
  if constexpr (NT == 192 || NT == 224) {
    if (res_stages > 0) {
      auto kernel = sparse_gemm_pair_kernel<NT, KB, kOutBf16Tma, true>;
      SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      SS_CUDA(cudaFuncGetAttributes(&attr, kernel));
      smem = PairResident<NT, KB>::smem_bytes(slabs);
      stages = res_stages;
      r->threads = kPairThreads; r->smem = smem; r->regs = attr.numRegs;
      r->local = static_cast<int>(attr.localSizeBytes); r->ctas_per_sm = 1;
      r->token_tile = NT; r->stages = stages; r->tmem_cols = kTmemCols;
      return SS_OK;
    }
  }
  if (split) {
    auto kernel = sparse_gemm_pair_kernel<NT, KB, kOutBf16TmaSplit>;
    SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes));
    SS_CUDA(cudaFuncGetAttributes(&attr, kernel));
  } else {
    auto kernel = sparse_gemm_pair_kernel<NT, KB, kOutBf16Tma>;
    SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes));
    SS_CUDA(cudaFuncGetAttributes(&attr, kernel));
  }
  r->threads = kPairThreads; r->smem = smem; r->regs = attr.numRegs;
  r->local = static_cast<int>(attr.localSizeBytes); r->ctas_per_sm = 1;
  r->token_tile = NT; r->stages = stages; r->tmem_cols = kTmemCols;
  return SS_OK;
}

// Resources of the kernel variant launch_gemm would use for an aligned BF16 output of this size.
int gemm_resources(int64_t m, int64_t n, int64_t pk, GemmResources* r) {
  DeviceInfo* dev = device_info();
  SS_REQUIRE(dev, SS_E_CUDA, "gemm: no current CUDA device");
  GemmArgs a{};
  a.m = m; a.n = n; a.pm = ceil_to(m, 32); a.pn = ceil_to(n, 32); a.pk = pk;
  a.out = nullptr; a.out_stride = ceil_to(n, 8);
  const Choice c = choose(a, dev->sms, true);
  const int slabs = static_cast<int>((pk / kBlockK + 1) / 2);
  switch (c.nt) {
    case 128: return pair_resources_t<128, 2>(r, 0, slabs, c.split);
    case 192: return pair_resources_t<192, 2>(r, c.res_stages, slabs, c.split);
    case 224: return pair_resources_t<224, 2>(r, c.res_stages, slabs, c.split);
    case 240: return pair_resources_t<240, 2>(r, 0, slabs, c.split);
    default:  return pair_resources_t<256, 2>(r, 0, slabs, c.split);
  }
}

}  // namespace ss

#ifdef SS_TIMELINE
// Development builds only (-DSS_TIMELINE): copies the per-tile time stamps to the host and clears them.
extern "C" int ss_timeline_read(long long* host, int count) {
  using namespace ss;
  const size_t total = sizeof(g_timeline) / sizeof(long long);
  SS_REQUIRE(host && count > 0 && static_cast<size_t>(count) <= total, SS_E_ARG, "timeline: bad arguments");
  SS_CUDA(cudaDeviceSynchronize());
  SS_CUDA(cudaMemcpyFromSymbol(host, g_timeline, static_cast<size_t>(count) * sizeof(long long)));
  void* p = nullptr;
  SS_CUDA(cudaGetSymbolAddress(&p, g_timeline));
  SS_CUDA(cudaMemset(p, 0, sizeof(g_timeline)));
  return SS_OK;
}
extern "C" int ss_profile_read(long long* host, int count) {
  using namespace ss;
  SS_REQUIRE(host && count > 0 && static_cast<size_t>(count) <= sizeof(g_profile) / sizeof(long long), SS_E_ARG, "profile: bad arguments");
  SS_CUDA(cudaDeviceSynchronize());
  SS_CUDA(cudaMemcpyFromSymbol(host, g_profile, static_cast<size_t>(count) * sizeof(long long)));
  return SS_OK;
}
#endif
