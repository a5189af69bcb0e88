// C-ABI entry points: argument validation, plan registry, device status word.
#include "ss_common.cuh"
#include <memory>
#include <mutex>
#include <unordered_map>
#include <string>

namespace ss {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

// One status word per device (each device that loads the module has its own copy).
__device__ uint32_t g_device_status = 0;

uint32_t* device_status_ptr() {
  static std::mutex mu;
  static std::unordered_map<int, uint32_t*> table;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  auto it = table.find(dev);
  if (it != table.end()) return it->second;
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
  table[dev] = static_cast<uint32_t*>(p);
  return static_cast<uint32_t*>(p);
}

namespace {

struct Plan {
  const int8_t* packed;
  const int32_t* meta;
  const float* sw;
  const float* bias;
  int64_t k, m, n, pn, pm, pk;
  int group, device;
  int8_t* q = nullptr;
  float* sa = nullptr;
  cudaStream_t owner = nullptr;
  bool has_owner = false;
  std::mutex mu;
  ~Plan() {
    if (q) cudaFree(q);
    if (sa) cudaFree(sa);
  }
};

struct Registry {
  std::mutex mu;
  int64_t next = 1;
  std::unordered_map<int64_t, std::shared_ptr<Plan>> plans;
};
Registry& registry() {
  static Registry* r = new Registry();
  return *r;
}
std::shared_ptr<Plan> find_plan(int64_t handle) {
  Registry& r = registry();
  std::lock_guard<std::mutex> lock(r.mu);
  auto it = r.plans.find(handle);
  return it == r.plans.end() ? nullptr : it->second;
}

int check_projection_shape(int64_t m, int64_t k, int64_t n, int64_t pn, int group, int64_t* pm,
                           int64_t* pk) {
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "group must be 4, 6 or 8 (got %d)", group);
  SS_REQUIRE(m > 0 && k > 0 && n > 0, SS_E_ARG, "positive m, k, n required");
  SS_REQUIRE(pn % 32 == 0 && pn >= n, SS_E_ARG, "pn must be a multiple of 32 and >= n");
  int64_t valid;
  ss_lifted_k(k, group, &valid, pk);
  *pm = ceil_to(m, 32);
  return SS_OK;
}

}  // namespace
}  // namespace ss

using namespace ss;

extern "C" const char* ss_last_error(void) { return g_error; }

extern "C" int ss_query(int device, int64_t* out, int n_out) {
  SS_REQUIRE(out && n_out >= 8, SS_E_ARG, "query: out must hold 8 values");
  for (int i = 0; i < n_out; ++i) out[i] = 0;
  out[0] = 1;
  out[1] = 100;
  out[6] = 512;
  out[7] = 192;
  if (device >= 0) {
    cudaDeviceProp p;
    SS_CUDA(cudaGetDeviceProperties(&p, device));
    out[2] = p.major;
    out[3] = p.minor;
    out[4] = p.multiProcessorCount;
    out[5] = static_cast<int64_t>(p.sharedMemPerBlockOptin);
  }
  return SS_OK;
}

extern "C" int ss_quantize_lift(const void* x, int64_t sx, int64_t m, int64_t k, int group,
                                int8_t* q, float* sa, void* stream) {
  return launch_quantize_lift(x, sx, m, k, group, q, sa, static_cast<cudaStream_t>(stream));
}

extern "C" int ss_gemm_run(const int8_t* q, const int8_t* packed, const int32_t* meta,
                           const float* sa, const float* sw, const float* bias,
                           const void* addend, int64_t addend_stride, void* out,
                           int64_t out_stride, int64_t m, int64_t n, int64_t pm, int64_t pn,
                           int64_t pk, void* stream) {
  GemmArgs a{q, packed, meta, sa, sw, bias, addend, addend_stride, out, out_stride,
             m, n, pm, pn, pk, false};
  return launch_gemm(a, static_cast<cudaStream_t>(stream));
}

extern "C" int ss_gemm_int32(const int8_t* q, const int8_t* packed, const int32_t* meta,
                             int32_t* acc, int64_t m, int64_t n, int64_t pm, int64_t pn,
                             int64_t pk, void* stream) {
  GemmArgs a{q, packed, meta, nullptr, nullptr, nullptr, nullptr, 0, acc, n,
             m, n, pm, pn, pk, true};
  return launch_gemm(a, static_cast<cudaStream_t>(stream));
}

extern "C" int ss_projection(const void* x, int64_t sx, int64_t m, int64_t k, int group,
                             const int8_t* packed, const int32_t* meta, const float* sw,
                             const float* bias, const void* addend, int64_t addend_stride,
                             int64_t n, int64_t pn, int8_t* q_scratch, float* sa_scratch,
                             void* out, int64_t out_stride, void* stream) {
  int64_t pm, pk;
  if (int rc = check_projection_shape(m, k, n, pn, group, &pm, &pk)) return rc;
  SS_REQUIRE(q_scratch && sa_scratch, SS_E_ARG, "projection: scratch buffers required");
  auto s = static_cast<cudaStream_t>(stream);
  if (int rc = launch_quantize_lift(x, sx, m, k, group, q_scratch, sa_scratch, s)) return rc;
  GemmArgs a{q_scratch, packed, meta, sa_scratch, sw, bias, addend, addend_stride, out,
             out_stride, m, n, pm, pn, pk, false};
  a.overlap_prologue = true;
  return launch_gemm(a, s);
}

extern "C" int ss_quantize_lift_fused(const void* x, int64_t sx, int64_t m, int64_t k, int group,
                                      int prologue, const void* shift, const void* scale,
                                      int64_t mod_stride, int64_t rows_per_batch, float eps,
                                      int8_t* q, float* sa, void* stream) {
  return launch_quantize_lift_fused(x, sx, m, k, group, prologue, shift, scale, mod_stride, rows_per_batch,
                                    eps, q, sa, static_cast<cudaStream_t>(stream));
}

extern "C" int ss_projection_fused(const void* x, int64_t sx, int64_t m, int64_t k, int group,
                                   int prologue, const void* shift, const void* scale,
                                   int64_t mod_stride, int64_t rows_per_batch, float eps,
                                   const int8_t* packed,
                                   const int32_t* meta, const float* sw, const float* bias,
                                   const void* addend, int64_t addend_stride,
                                   const void* gate, int64_t gate_stride, int64_t n, int64_t pn,
                                   int8_t* q_scratch, float* sa_scratch, void* out,
                                   int64_t out_stride, void* stream) {
  int64_t pm, pk;
  if (int rc = check_projection_shape(m, k, n, pn, group, &pm, &pk)) return rc;
  SS_REQUIRE(q_scratch && sa_scratch, SS_E_ARG, "projection: scratch buffers required");
  auto s = static_cast<cudaStream_t>(stream);
  if (int rc = launch_quantize_lift_fused(x, sx, m, k, group, prologue, shift, scale, mod_stride,
                                          rows_per_batch, eps, q_scratch, sa_scratch, s)) return rc;
  GemmArgs a{q_scratch, packed, meta, sa_scratch, sw, bias, addend, addend_stride, out,
             out_stride, m, n, pm, pn, pk, false};
  a.overlap_prologue = true;
  a.gate = gate;
  a.gate_stride = gate_stride;
  a.rows_per_batch = rows_per_batch;
  return launch_gemm(a, s);
}

extern "C" int ss_projection_peers(const void* x, int64_t sx, int64_t m, int64_t k, int group,
                                   const int8_t* packed, const int32_t* meta, const float* sw,
                                   const float* bias, int64_t n, int64_t pn, int8_t* q_scratch,
                                   float* sa_scratch, const void* const* destinations, int count,
                                   int64_t out_stride, void* stream) {
  int64_t pm, pk;
  if (int rc = check_projection_shape(m, k, n, pn, group, &pm, &pk)) return rc;
  SS_REQUIRE(q_scratch && sa_scratch, SS_E_ARG, "projection: scratch buffers required");
  SS_REQUIRE(destinations && count >= 1 && count <= kMaxPeers, SS_E_ARG,
             "projection: 1..%d destination pointers required", kMaxPeers);
  auto s = static_cast<cudaStream_t>(stream);
  if (int rc = launch_quantize_lift(x, sx, m, k, group, q_scratch, sa_scratch, s)) return rc;
  GemmArgs a{q_scratch, packed, meta, sa_scratch, sw, bias, nullptr, 0, nullptr, out_stride,
             m, n, pm, pn, pk, false};
  a.overlap_prologue = true;
  a.peer_count = count;
  for (int g = 0; g < count; ++g) a.peer_out[g] = destinations[g];
  return launch_gemm(a, s);
}

extern "C" int ss_plan_create(const int8_t* packed, const int32_t* meta, const float* sw,
                              const float* bias, int64_t k, int64_t m, int64_t n, int64_t pn,
                              int group, int64_t* handle) {
  SS_REQUIRE(handle, SS_E_ARG, "plan_create: handle pointer required");
  SS_REQUIRE(packed && meta && sw, SS_E_ARG, "plan_create: null pointer");
  auto plan = std::make_shared<Plan>();
  if (int rc = check_projection_shape(m, k, n, pn, group, &plan->pm, &plan->pk)) return rc;
  plan->packed = packed; plan->meta = meta; plan->sw = sw; plan->bias = bias;
  plan->k = k; plan->m = m; plan->n = n; plan->pn = pn; plan->group = group;
  SS_CUDA(cudaGetDevice(&plan->device));
  SS_CUDA(cudaMalloc(&plan->q, static_cast<size_t>(plan->pm) * plan->pk));
  SS_CUDA(cudaMalloc(&plan->sa, static_cast<size_t>(plan->pm) * sizeof(float)));
  Registry& r = registry();
  std::lock_guard<std::mutex> lock(r.mu);
  *handle = r.next++;
  r.plans[*handle] = plan;
  return SS_OK;
}

extern "C" int ss_plan_run(int64_t handle, const void* x, int64_t sx, int8_t* q_scratch,
                           float* sa_scratch, void* out, int64_t out_stride, void* stream) {
  auto plan = find_plan(handle);
  SS_REQUIRE(plan, SS_E_HANDLE, "prepared handle %lld absent", (long long)handle);
  int dev = 0;
  SS_CUDA(cudaGetDevice(&dev));
  SS_REQUIRE(dev == plan->device, SS_E_ARG, "plan belongs to device %d, current device is %d",
             plan->device, dev);
  auto s = static_cast<cudaStream_t>(stream);
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  SS_CUDA(cudaStreamIsCapturing(s, &capture));
  std::unique_lock<std::mutex> lock(plan->mu);
  const bool first = !plan->has_owner;
  const bool resident = capture == cudaStreamCaptureStatusNone && (first || plan->owner == s);
  int8_t* q = q_scratch;
  float* sa = sa_scratch;
  if (!q || !sa) {
    SS_REQUIRE(resident, SS_E_ARG,
               "plan_run: caller scratch required on a foreign stream or during stream capture");
    q = plan->q;
    sa = plan->sa;
    plan->owner = s;
    plan->has_owner = true;
  }
  if (int rc = launch_quantize_lift(x, sx, plan->m, plan->k, plan->group, q, sa, s)) return rc;
  GemmArgs a{q, plan->packed, plan->meta, sa, plan->sw, plan->bias, nullptr, 0, out, out_stride,
             plan->m, plan->n, plan->pm, plan->pn, plan->pk, false};
  a.overlap_prologue = true;
  return launch_gemm(a, s);
}

extern "C" int ss_plan_release(int64_t handle) {
  std::shared_ptr<Plan> plan;
  {
    Registry& r = registry();
    std::lock_guard<std::mutex> lock(r.mu);
    auto it = r.plans.find(handle);
    if (it == r.plans.end()) return SS_OK;
    plan = it->second;
    r.plans.erase(it);
  }
  int prev = 0;
  SS_CUDA(cudaGetDevice(&prev));
  SS_CUDA(cudaSetDevice(plan->device));
  if (plan->has_owner) cudaStreamSynchronize(plan->owner);
  plan.reset();
  SS_CUDA(cudaSetDevice(prev));
  return SS_OK;
}

extern "C" int ss_plan_resources(int64_t handle, int64_t* out, int n_out) {
  auto plan = find_plan(handle);
  SS_REQUIRE(plan, SS_E_HANDLE, "prepared handle %lld absent", (long long)handle);
  SS_REQUIRE(out && n_out >= 8, SS_E_ARG, "plan_resources: out must hold 8 values");
  GemmResources r;
  if (int rc = gemm_resources(plan->m, plan->n, plan->pk, &r)) return rc;
  out[0] = r.threads; out[1] = r.smem; out[2] = r.regs; out[3] = r.local;
  out[4] = r.ctas_per_sm; out[5] = r.token_tile; out[6] = r.stages; out[7] = r.tmem_cols;
  return SS_OK;
}

extern "C" int ss_gemm_resources(int64_t m, int64_t n, int64_t pk, int64_t* out, int n_out) {
  SS_REQUIRE(out && n_out >= 8, SS_E_ARG, "gemm_resources: out must hold 8 values");
  SS_REQUIRE(m > 0 && n > 0 && pk > 0 && pk % 128 == 0, SS_E_ARG, "gemm_resources: invalid shape");
  GemmResources r;
  if (int rc = gemm_resources(m, n, pk, &r)) return rc;
  out[0] = r.threads; out[1] = r.smem; out[2] = r.regs; out[3] = r.local;
  out[4] = r.ctas_per_sm; out[5] = r.token_tile; out[6] = r.stages; out[7] = r.tmem_cols;
  return SS_OK;
}

extern "C" int ss_device_status(void* stream, int32_t* status) {
  SS_REQUIRE(status, SS_E_ARG, "device_status: status pointer required");
  SS_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  uint32_t* p = device_status_ptr();
  SS_REQUIRE(p, SS_E_CUDA, "device status word unavailable");
  uint32_t v = 0;
  SS_CUDA(cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost));
  if (v) {
    SS_CUDA(cudaMemset(p, 0, sizeof(v)));
    // a launch that gave up may have left sums of shared tiles behind
    if (int rc = reset_split_workspace()) return rc;
  }
  *status = static_cast<int32_t>(v);
  SS_REQUIRE(v == 0, SS_E_DEVICE,
             "a kernel gave up on a bounded wait (status 0x%x:%s%s%s%s); results of the launches since the "
             "last check are not to be trusted",
             v, (v & kStatusProducerTimeout) ? " TMA producer" : "", (v & kStatusMmaTimeout) ? " MMA issuer" : "",
             (v & kStatusEpilogueTimeout) ? " epilogue" : "", (v & kStatusProbeTimeout) ? " wait-limit probe" : "");
  return SS_OK;
}

namespace {
struct OptionField { const char* name; int Options::*field; };
const OptionField kOptionFields[] = {
    {"token_tile", &Options::token_tile}, {"wide_cp", &Options::wide_cp}, {"meta_warp", &Options::meta_warp},
    {"store", &Options::store},           {"resident", &Options::resident}, {"pdl", &Options::pdl},
    {"split", &Options::split},
};
}  // namespace

extern "C" int ss_set_option(const char* name, int64_t value) {
  SS_REQUIRE(name, SS_E_ARG, "set_option: name required");
  Options& opt = options();
  if (std::string(name) == "wait_ns") {
    SS_REQUIRE(value > 0, SS_E_ARG, "set_option: wait_ns must be positive");
    opt.wait_ns = static_cast<unsigned long long>(value);
    return SS_OK;
  }
  for (const OptionField& f : kOptionFields)
    if (std::string(name) == f.name) {
      opt.*(f.field) = static_cast<int>(value);
      return SS_OK;
    }
  set_error("set_option: unknown option '%s'", name);
  return SS_E_ARG;
}

extern "C" int ss_get_option(const char* name, int64_t* value) {
  SS_REQUIRE(name && value, SS_E_ARG, "get_option: name and value pointer required");
  const Options& opt = options();
  if (std::string(name) == "wait_ns") {
    *value = static_cast<int64_t>(opt.wait_ns);
    return SS_OK;
  }
  if (std::string(name) == "split_launches") {
    *value = static_cast<int64_t>(split_launch_count());
    return SS_OK;
  }
  for (const OptionField& f : kOptionFields)
    if (std::string(name) == f.name) {
      *value = opt.*(f.field);
      return SS_OK;
    }
  set_error("get_option: unknown option '%s'", name);
  return SS_E_ARG;
}
