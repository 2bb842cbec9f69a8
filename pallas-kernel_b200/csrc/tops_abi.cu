// extern "C" entry points: validation, workspace carving, kernel selection.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "elementwise.cuh"
#include "gla_generic.cuh"
#include "gla_sm100.cuh"
#include "kda.cuh"
#include "kda_sm100.cuh"
#include "recurrent.cuh"

namespace tops {
static std::atomic<int64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static std::mutex g_err_mu;
static char g_err_text[256] = "";
void record_cuda_error(int code, const char* where) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  snprintf(g_err_text, sizeof g_err_text, "%s: %s (%d)", where, cudaGetErrorString((cudaError_t)code), code);
}

namespace {
struct ProfRecord { const char* label; cudaEvent_t start, stop; };
std::atomic<int> g_prof_on{0};
std::mutex g_prof_mu;
std::vector<ProfRecord> g_prof;
constexpr size_t kMaxProfRecords = 1 << 16;
}  // namespace

KernelScope::KernelScope(const char* label, cudaStream_t s) : slot(-1), st(s) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof.size() >= kMaxProfRecords) return;
  ProfRecord r{label, nullptr, nullptr};
  if (cudaEventCreate(&r.start) != cudaSuccess || cudaEventCreate(&r.stop) != cudaSuccess) return;
  cudaEventRecord(r.start, st);
  g_prof.push_back(r);
  slot = (int)g_prof.size() - 1;
}
KernelScope::~KernelScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  cudaEventRecord(g_prof[slot].stop, st);
}

namespace {

struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(reinterpret_cast<char*>(p)) {}
  template <class T> T* take(size_t count) {
    T* r = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += align_up(count * sizeof(T));
    return r;
  }
};

bool valid_dtype(int dt) { return dt == TOPS_F32 || dt == TOPS_BF16 || dt == TOPS_F16; }

int check_problem(const tops_chunk_problem& pb) {
  if (pb.B < 1 || pb.T < 1 || pb.H < 1 || pb.K < 1 || pb.V < 1) return TOPS_E_BAD_SHAPE;
  if (pb.chunk != 16 && pb.chunk != 32 && pb.chunk != 64) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(pb.dtype) || !valid_dtype(pb.gate_dtype)) return TOPS_E_BAD_DTYPE;
  if (pb.gate_kind < TOPS_GATE_NONE || pb.gate_kind > TOPS_GATE_GAMMA) return TOPS_E_BAD_SHAPE;
  if (pb.gate_kind == TOPS_GATE_GAMMA && pb.gate_dtype != TOPS_F32) return TOPS_E_BAD_DTYPE;
  if (pb.cu_seqlens) {
    if (pb.B != 1 || pb.N < 1 || pb.cu_seqlens_host == nullptr) return TOPS_E_BAD_SHAPE;
    if (pb.cu_seqlens_host[0] != 0 || pb.cu_seqlens_host[pb.N] != pb.T) return TOPS_E_BAD_SHAPE;
    for (int n = 0; n < pb.N; ++n)
      if (pb.cu_seqlens_host[n + 1] <= pb.cu_seqlens_host[n]) return TOPS_E_BAD_SHAPE;
  }
  return TOPS_OK;
}

int count_chunks(const tops_chunk_problem& pb) {
  if (!pb.cu_seqlens) return pb.B * cdiv(pb.T, pb.chunk);
  int tot = 0;
  for (int n = 0; n < pb.N; ++n) tot += cdiv(pb.cu_seqlens_host[n + 1] - pb.cu_seqlens_host[n], pb.chunk);
  return tot;
}

size_t gate_elems(const tops_chunk_problem& pb) {
  size_t tok = (size_t)pb.B * pb.T * pb.H;
  if (pb.gate_kind == TOPS_GATE_PER_CHANNEL) return tok * pb.K;
  if (pb.gate_kind == TOPS_GATE_SCALAR) return tok;
  return 0;
}

// Fills Problem (minus gcum) and the packed-batch tables carved from `cv`.
int make_problem(const tops_chunk_problem& in, Carver& cv, cudaStream_t st, Problem* out, bool launch) {
  Problem pb{};
  pb.H = in.H; pb.K = in.K; pb.V = in.V; pb.dtype = in.dtype; pb.gate_kind = in.gate_kind; pb.scale = in.scale;
  pb.total_chunks = count_chunks(in);
  pb.m.T = in.T; pb.m.C = in.chunk;
  if (in.cu_seqlens) {
    int32_t* cs = cv.take<int32_t>(in.N + 1);
    int32_t* chunk_seq = cv.take<int32_t>(pb.total_chunks);
    pb.m.cu = in.cu_seqlens; pb.m.cs = cs; pb.m.chunk_seq = chunk_seq; pb.m.N = in.N; pb.m.NT = pb.total_chunks;
    if (launch) {
      int rc = generic::launch_prepare_chunks(in.cu_seqlens, in.N, in.chunk, cs, chunk_seq, st);
      if (rc) return rc;
    }
  } else {
    pb.m.cu = nullptr; pb.m.cs = nullptr; pb.m.chunk_seq = nullptr; pb.m.N = in.B; pb.m.NT = cdiv(in.T, in.chunk);
  }
  *out = pb;
  return TOPS_OK;
}

size_t state_elems(const tops_chunk_problem& pb) {
  return (size_t)count_chunks(pb) * pb.H * pb.K * pb.V;
}

bool use_sm100(const tops_chunk_problem& pb) {
  if (pb.impl == TOPS_IMPL_GENERIC) return false;
  return sm100::supported(pb);
}

}  // namespace
}  // namespace tops

using namespace tops;

extern "C" const char* tops_b200_strerror(int code) {
  switch (code) {
    case TOPS_OK: return "ok";
    case TOPS_E_BAD_SHAPE: return "bad shape or unsupported dimension";
    case TOPS_E_BAD_DTYPE: return "bad dtype";
    case TOPS_E_NULL: return "required pointer is NULL";
    case TOPS_E_WORKSPACE: return "workspace missing or too small";
    case TOPS_E_CUDA: return "CUDA call failed";
    case TOPS_E_UNSUPPORTED: return "no kernel covers this request";
    case TOPS_E_ALIGN: return "pointer is not 16-byte aligned";
    case TOPS_E_STATIC_LIMIT: return "problem needs more scratch than the built-in static buffer holds";
    default: return "unknown error";
  }
}

extern "C" int64_t tops_b200_launch_count(void) { return g_launches.load(); }

extern "C" int tops_b200_last_cuda_error(char* buf, size_t cap) {
  if (!buf || cap == 0) return TOPS_E_NULL;
  std::lock_guard<std::mutex> lk(g_err_mu);
  snprintf(buf, cap, "%s", g_err_text);
  return TOPS_OK;
}

extern "C" int tops_b200_chunk_selected_impl(const tops_chunk_problem* pb) {
  if (!pb || check_problem(*pb)) return TOPS_IMPL_GENERIC;
  return use_sm100(*pb) ? TOPS_IMPL_SM100 : TOPS_IMPL_GENERIC;
}

extern "C" int tops_b200_device_error(int* out) {
  if (!out) return TOPS_E_NULL;
  int a = 0, b = 0;
  int rc = sm100::device_error(&a);
  if (rc == TOPS_OK) rc = sm100::kda_device_error(&b);
  *out = a ? a : b;
  return rc;
}

extern "C" int tops_b200_device_error_set(int code) {
  int rc = sm100::device_error_set(code);
  return rc ? rc : sm100::kda_device_error_set(code);
}

extern "C" int tops_b200_device_error_reset(void) { return tops_b200_device_error_set(0); }

extern "C" int tops_b200_test_skip_load(int chunk) {
  sm100::test_skip_load(chunk);
  return TOPS_OK;
}

extern "C" int tops_b200_profile_enable(int on) {
  g_prof_on.store(on ? 1 : 0);
  return TOPS_OK;
}

extern "C" int tops_b200_profile_read(char* buf, size_t cap) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  std::map<std::string, std::pair<int, double>> agg;
  int rc = TOPS_OK;
  for (auto& r : g_prof) {
    float ms = 0.f;
    if (cudaEventSynchronize(r.stop) != cudaSuccess || cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess)
      rc = TOPS_E_CUDA;
    auto& a = agg[r.label];
    a.first += 1;
    a.second += ms;
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  g_prof.clear();
  size_t off = 0;
  if (buf && cap) buf[0] = 0;
  for (auto& kv : agg) {
    char line[256];
    int n = snprintf(line, sizeof line, "%s %d %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
    if (buf && off + n + 1 <= cap) { memcpy(buf + off, line, n + 1); off += n; }
  }
  return rc;
}

extern "C" int tops_b200_chunk_local_cumsum(const tops_cumsum_params* p, void* stream) {
  if (!p || !p->g || !p->out) return TOPS_E_NULL;
  if (p->B < 1 || p->T < 1 || p->H < 1 || p->D < 1) return TOPS_E_BAD_SHAPE;
  if (p->chunk < 1 || (p->chunk & (p->chunk - 1))) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(p->dtype)) return TOPS_E_BAD_DTYPE;
  if (p->cu_seqlens) return TOPS_E_UNSUPPORTED;  // packed batches: the fused chunk entry points do their own cumsum
  SeqMap m{};
  m.N = p->B; m.T = p->T; m.C = p->chunk; m.NT = cdiv(p->T, p->chunk);
  return generic::launch_cumsum(m, p->H, p->D, p->dtype, p->reverse, p->g, p->out, p->B * m.NT,
                                (cudaStream_t)stream);
}

extern "C" int tops_b200_chunk_fwd_h(const tops_fwd_h_params* p, void* stream) {
  if (!p || !p->k || !p->v) return TOPS_E_NULL;
  int rc = check_problem(p->pb);
  if (rc) return rc;
  if (p->pb.cu_seqlens) return TOPS_E_UNSUPPORTED;
  if (p->pb.gate_kind != TOPS_GATE_NONE && !p->g_cumsum) return TOPS_E_NULL;
  if (p->h && p->h_dtype != TOPS_F32 && p->h_dtype != p->pb.dtype) return TOPS_E_BAD_DTYPE;
  Carver cv(nullptr);
  Problem pb;
  if ((rc = make_problem(p->pb, cv, (cudaStream_t)stream, &pb, true))) return rc;
  pb.gcum = p->g_cumsum;
  return generic::launch_scan(pb, false, p->k, p->v, p->h0, p->h, p->h_dtype == TOPS_F32, p->ht,
                              (cudaStream_t)stream);
}

extern "C" int tops_b200_chunk_bwd_dh(const tops_bwd_dh_params* p, void* stream) {
  if (!p || !p->q || !p->do_) return TOPS_E_NULL;
  int rc = check_problem(p->pb);
  if (rc) return rc;
  if (p->pb.cu_seqlens) return TOPS_E_UNSUPPORTED;
  if (p->pb.gate_kind != TOPS_GATE_NONE && !p->g_cumsum) return TOPS_E_NULL;
  Carver cv(nullptr);
  Problem pb;
  if ((rc = make_problem(p->pb, cv, (cudaStream_t)stream, &pb, true))) return rc;
  pb.gcum = p->g_cumsum;
  return generic::launch_scan(pb, true, p->q, p->do_, p->dht, p->dh, 1, p->dh0, (cudaStream_t)stream);
}

// ---- forward ----------------------------------------------------------------
static size_t fwd_layout(const tops_chunk_fwd_params* p, void* ws, cudaStream_t st, bool launch, Problem* pb,
                         float** gcum, void** h, int* rc_out) {
  Carver cv(ws);
  int rc = make_problem(p->pb, cv, st, pb, launch);
  if (rc_out) *rc_out = rc;
  size_t ge = gate_elems(p->pb);
  float* g = (p->g_cumsum_out || ge == 0) ? p->g_cumsum_out : cv.take<float>(ge);
  if (p->g_cumsum_out == nullptr && ge != 0 && ws == nullptr) g = nullptr;
  char* hh = p->h_out ? reinterpret_cast<char*>(p->h_out)
                      : reinterpret_cast<char*>(cv.take<char>(state_elems(p->pb) * dtype_size(p->pb.dtype)));
  if (gcum) *gcum = g;
  if (h) *h = hh;
  return cv.off;
}

extern "C" size_t tops_b200_chunk_fwd_workspace_bytes(const tops_chunk_fwd_params* p) {
  if (!p || check_problem(p->pb)) return 0;
  if (use_sm100(p->pb) && !p->g_cumsum_out && !p->A_out && !p->h_out) return sm100::fwd_workspace_bytes(*p);
  Problem pb;
  return fwd_layout(p, nullptr, nullptr, false, &pb, nullptr, nullptr, nullptr) + 256;
}

extern "C" int tops_b200_chunk_gla_fwd(const tops_chunk_fwd_params* p, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->o) return TOPS_E_NULL;
  int rc = check_problem(p->pb);
  if (rc) return rc;
  if (p->pb.gate_kind != TOPS_GATE_NONE && !p->g) return TOPS_E_NULL;
  if (p->pb.impl == TOPS_IMPL_SM100 && !sm100::supported(p->pb)) return TOPS_E_UNSUPPORTED;
  if (!workspace || workspace_bytes < tops_b200_chunk_fwd_workspace_bytes(p)) return TOPS_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (use_sm100(p->pb) && !p->g_cumsum_out && !p->A_out && !p->h_out) return sm100::chunk_fwd(*p, workspace, workspace_bytes, st);

  Problem pb;
  float* gcum = nullptr;
  void* h = nullptr;
  fwd_layout(p, workspace, st, true, &pb, &gcum, &h, &rc);
  if (rc) return rc;
  if (p->pb.gate_kind == TOPS_GATE_PER_CHANNEL || p->pb.gate_kind == TOPS_GATE_SCALAR) {
    int D = p->pb.gate_kind == TOPS_GATE_PER_CHANNEL ? p->pb.K : 1;
    if ((rc = generic::launch_cumsum(pb.m, pb.H, D, p->pb.gate_dtype, 0, p->g, gcum, pb.total_chunks, st))) return rc;
    pb.gcum = gcum;
  } else if (p->pb.gate_kind == TOPS_GATE_GAMMA) {
    pb.gcum = reinterpret_cast<const float*>(p->g);
  }
  if ((rc = generic::launch_scan(pb, false, p->k, p->v, p->h0, h, 0, p->ht, st))) return rc;
  int round_A = p->pb.gate_kind == TOPS_GATE_PER_CHANNEL || p->pb.gate_kind == TOPS_GATE_NONE;
  return generic::launch_fwd_o(pb, p->q, p->k, p->v, h, 0, p->o, p->A_out, round_A, st);
}

// ---- forward on the library's own scratch ---------------------------------------
// Scratch for callers that can neither allocate device memory nor pass a
// workspace.  In host code this name is only a handle for the runtime: the
// device address has to be looked up with cudaGetSymbolAddress, per device.
static __device__ __align__(256) unsigned char g_static_scratch[TOPS_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the current device (looked up once per device).
int static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TOPS_E_CUDA;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return TOPS_E_CUDA;
    }
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return TOPS_OK;
}
}  // namespace

extern "C" int tops_b200_chunk_gla_fwd_static(const tops_chunk_fwd_params* p, void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->o) return TOPS_E_NULL;
  int rc = check_problem(p->pb);
  if (rc) return rc;
  const size_t need = tops_b200_chunk_fwd_workspace_bytes(p);
  if (need == 0 || need > TOPS_STATIC_SCRATCH_BYTES) return TOPS_E_STATIC_LIMIT;
  void* scratch = nullptr;
  if ((rc = static_scratch(&scratch))) return rc;
  return tops_b200_chunk_gla_fwd(p, scratch, TOPS_STATIC_SCRATCH_BYTES, stream);
}

// ---- backward ---------------------------------------------------------------
struct BwdLayout {
  float *gcum, *h, *dh, *A, *dA, *dg_part;
  size_t dg_stride;
  int tilesK;
};

static size_t bwd_layout(const tops_chunk_bwd_params* p, void* ws, cudaStream_t st, bool launch, Problem* pb,
                         BwdLayout* L, int* rc_out) {
  Carver cv(ws);
  int rc = make_problem(p->pb, cv, st, pb, launch);
  if (rc_out) *rc_out = rc;
  BwdLayout l{};
  size_t ge = gate_elems(p->pb);
  l.gcum = ge ? cv.take<float>(ge) : nullptr;
  size_t se = state_elems(p->pb);
  l.h = cv.take<float>(se);
  l.dh = cv.take<float>(se);
  size_t ae = (size_t)pb->total_chunks * p->pb.H * p->pb.chunk * p->pb.chunk;
  l.A = cv.take<float>(ae);
  l.dA = cv.take<float>(ae);
  l.tilesK = cdiv(p->pb.K, 64);
  l.dg_stride = (size_t)p->pb.B * p->pb.T * p->pb.H;
  l.dg_part = p->pb.gate_kind == TOPS_GATE_SCALAR ? cv.take<float>(l.dg_stride * l.tilesK) : nullptr;
  if (L) *L = l;
  return cv.off;
}

extern "C" size_t tops_b200_chunk_bwd_workspace_bytes(const tops_chunk_bwd_params* p) {
  if (!p || check_problem(p->pb)) return 0;
  if (use_sm100(p->pb) && sm100::bwd_dtypes_ok(*p)) return sm100::bwd_workspace_bytes(*p);
  Problem pb;
  return bwd_layout(p, nullptr, nullptr, false, &pb, nullptr, nullptr) + 256;
}

extern "C" int tops_b200_chunk_gla_bwd(const tops_chunk_bwd_params* p, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->do_ || !p->dq || !p->dk || !p->dv) return TOPS_E_NULL;
  int rc = check_problem(p->pb);
  if (rc) return rc;
  if (p->pb.gate_kind != TOPS_GATE_NONE && !p->g) return TOPS_E_NULL;
  if (!valid_dtype(p->grad_dtype)) return TOPS_E_BAD_DTYPE;
  if (p->pb.impl == TOPS_IMPL_SM100 && !sm100::supported(p->pb)) return TOPS_E_UNSUPPORTED;
  if (!workspace || workspace_bytes < tops_b200_chunk_bwd_workspace_bytes(p)) return TOPS_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (use_sm100(p->pb) && sm100::bwd_dtypes_ok(*p)) return sm100::chunk_bwd(*p, workspace, workspace_bytes, st);
  if (p->dg_dtype != TOPS_F32) return TOPS_E_UNSUPPORTED;   // the generic kernels write fp32 dg per gate element

  Problem pb;
  BwdLayout L;
  bwd_layout(p, workspace, st, true, &pb, &L, &rc);
  if (rc) return rc;
  const int kind = p->pb.gate_kind;
  if (kind == TOPS_GATE_PER_CHANNEL || kind == TOPS_GATE_SCALAR) {
    int D = kind == TOPS_GATE_PER_CHANNEL ? p->pb.K : 1;
    if ((rc = generic::launch_cumsum(pb.m, pb.H, D, p->pb.gate_dtype, 0, p->g, L.gcum, pb.total_chunks, st))) return rc;
    pb.gcum = L.gcum;
  } else if (kind == TOPS_GATE_GAMMA) {
    pb.gcum = reinterpret_cast<const float*>(p->g);
  }
  if ((rc = generic::launch_scan(pb, false, p->k, p->v, p->h0, L.h, 1, nullptr, st))) return rc;
  if ((rc = generic::launch_scan(pb, true, p->q, p->do_, p->dht, L.dh, 1, p->dh0, st))) return rc;
  BwdBuffers b{};
  b.q = p->q; b.k = p->k; b.v = p->v; b.do_ = p->do_; b.A = L.A; b.dA = L.dA; b.h = L.h; b.dh = L.dh;
  b.dq = p->dq; b.dk = p->dk; b.dv = p->dv; b.grad_dtype = p->grad_dtype;
  b.dg_stage = nullptr; b.dg_tile_stride = 0;
  if (p->dg && kind == TOPS_GATE_PER_CHANNEL) b.dg_stage = reinterpret_cast<float*>(p->dg);
  if (p->dg && kind == TOPS_GATE_SCALAR) { b.dg_stage = L.dg_part; b.dg_tile_stride = L.dg_stride; }
  if ((rc = generic::launch_bwd(pb, b, st))) return rc;
  if (p->dg && kind == TOPS_GATE_SCALAR)
    return generic::launch_sum_partials(L.dg_part, L.dg_stride, L.tilesK, reinterpret_cast<float*>(p->dg), L.dg_stride, st);
  return TOPS_OK;
}

// ---- recurrent --------------------------------------------------------------
extern "C" int tops_b200_fused_recurrent_gla_fwd(const tops_recurrent_fwd_params* p, void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->o) return TOPS_E_NULL;
  if (p->B < 1 || p->T < 1 || p->H < 1 || p->K < 1 || p->V < 1) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(p->dtype) || !valid_dtype(p->gate_dtype) || !valid_dtype(p->o_dtype)) return TOPS_E_BAD_DTYPE;
  if (p->cu_seqlens && (p->B != 1 || p->N < 1)) return TOPS_E_BAD_SHAPE;
  return recurrent::fwd(*p, (cudaStream_t)stream);
}

extern "C" size_t tops_b200_fused_recurrent_gla_bwd_workspace_bytes(const tops_recurrent_bwd_params* p) {
  if (!p) return 0;
  return recurrent::bwd_workspace_bytes(*p);
}

extern "C" int tops_b200_fused_recurrent_gla_bwd(const tops_recurrent_bwd_params* p, void* workspace,
                                                 size_t workspace_bytes, void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->do_ || !p->dq || !p->dk || !p->dv) return TOPS_E_NULL;
  if (p->B < 1 || p->T < 1 || p->H < 1 || p->K < 1 || p->V < 1) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(p->dtype) || !valid_dtype(p->gate_dtype)) return TOPS_E_BAD_DTYPE;
  if (p->gv && !p->o) return TOPS_E_NULL;
  if (p->cu_seqlens && (p->B != 1 || p->N < 1)) return TOPS_E_BAD_SHAPE;
  if (!workspace || workspace_bytes < recurrent::bwd_workspace_bytes(*p)) return TOPS_E_WORKSPACE;
  return recurrent::bwd(*p, workspace, (cudaStream_t)stream);
}

// ---- KDA ----------------------------------------------------------------------
extern "C" int tops_b200_kda_fwd(const tops_kda_fwd_params* p, void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->g || !p->beta || !p->o) return TOPS_E_NULL;
  if (p->B < 1 || p->T < 1 || p->H < 1 || p->K < 1 || p->V < 1 || p->K > 256) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(p->dtype) || !valid_dtype(p->gate_dtype)) return TOPS_E_BAD_DTYPE;
  return kda::fwd(*p, (cudaStream_t)stream);
}

extern "C" int tops_b200_chunk_kda_supported(const tops_chunk_kda_fwd_params* p) {
  if (!p || p->B < 1 || p->T < 1 || p->H < 1) return 0;
  return sm100::kda_supported(*p) ? 1 : 0;
}

extern "C" int tops_b200_chunk_kda_fwd(const tops_chunk_kda_fwd_params* p, void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->g || !p->beta || !p->o) return TOPS_E_NULL;
  if (p->B < 1 || p->T < 1 || p->H < 1 || p->K < 1 || p->V < 1) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(p->dtype) || !valid_dtype(p->gate_dtype)) return TOPS_E_BAD_DTYPE;
  if (!sm100::kda_supported(*p)) return TOPS_E_UNSUPPORTED;
  return sm100::kda_chunk_fwd(*p, (cudaStream_t)stream);
}

extern "C" size_t tops_b200_chunk_kda_bwd_workspace_bytes(const tops_chunk_kda_bwd_params* p) {
  if (!p || p->B < 1 || p->T < 1 || p->H < 1 || !sm100::kda_bwd_supported(*p)) return 0;
  return sm100::kda_chunk_bwd_workspace_bytes(*p);
}

extern "C" int tops_b200_chunk_kda_bwd(const tops_chunk_kda_bwd_params* p, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->g || !p->beta || !p->do_ || !p->saved_h || !p->saved_vnew || !p->saved_T ||
      !p->saved_R || !p->dv)
    return TOPS_E_NULL;
  {   // dq, dk, dg, dbeta: all four, or none (state gradient only, which must then be asked for)
    const int given = !!p->dq + !!p->dk + !!p->dg + !!p->dbeta;
    if ((given != 0 && given != 4) || (given == 0 && !p->dh0)) return TOPS_E_NULL;
  }
  if (p->B < 1 || p->T < 1 || p->H < 1 || p->K < 1 || p->V < 1) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(p->dtype) || !valid_dtype(p->gate_dtype) || !valid_dtype(p->grad_dtype)) return TOPS_E_BAD_DTYPE;
  if (!sm100::kda_bwd_supported(*p)) return TOPS_E_UNSUPPORTED;
  if (!workspace || workspace_bytes < sm100::kda_chunk_bwd_workspace_bytes(*p)) return TOPS_E_WORKSPACE;
  return sm100::kda_chunk_bwd(*p, workspace, (cudaStream_t)stream);
}

extern "C" size_t tops_b200_kda_bwd_workspace_bytes(const tops_kda_bwd_params* p) {
  return p ? kda::bwd_workspace_bytes(*p) : 0;
}

extern "C" int tops_b200_kda_bwd(const tops_kda_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (!p || !p->q || !p->k || !p->v || !p->g || !p->beta || !p->do_ || !p->dq || !p->dk || !p->dv || !p->dg ||
      !p->dbeta)
    return TOPS_E_NULL;
  if (p->B < 1 || p->T < 1 || p->H < 1 || p->K < 1 || p->V < 1 || p->K > 128 || p->V > 128) return TOPS_E_BAD_SHAPE;
  if (!valid_dtype(p->dtype) || !valid_dtype(p->gate_dtype)) return TOPS_E_BAD_DTYPE;
  if (!workspace || workspace_bytes < kda::bwd_workspace_bytes(*p)) return TOPS_E_WORKSPACE;
  return kda::bwd(*p, workspace, (cudaStream_t)stream);
}

// ---- gate activations and row normalisations -------------------------------------
extern "C" int tops_b200_gate_act_fwd(const tops_gate_act_params* p, void* stream) {
  if (!p || !p->g || !p->out) return TOPS_E_NULL;
  if (!valid_dtype(p->dtype) || !valid_dtype(p->out_dtype)) return TOPS_E_BAD_DTYPE;
  int rc = elementwise::gate_check(*p);
  return rc ? rc : elementwise::gate_fwd(*p, (cudaStream_t)stream);
}

extern "C" size_t tops_b200_gate_act_bwd_workspace_bytes(const tops_gate_act_bwd_params* p) {
  if (!p || p->fwd.rows < 1 || p->fwd.H < 1 || p->fwd.K < 1) return 0;
  return elementwise::gate_bwd_workspace_bytes(*p);
}

extern "C" int tops_b200_gate_act_bwd(const tops_gate_act_bwd_params* p, void* workspace, size_t workspace_bytes,
                                      void* stream) {
  if (!p || !p->fwd.g || !p->dy || !p->dg) return TOPS_E_NULL;
  if (!valid_dtype(p->fwd.dtype) || !valid_dtype(p->dy_dtype)) return TOPS_E_BAD_DTYPE;
  tops_gate_act_params f = p->fwd;
  f.out = p->dg;   // (only checked for alignment)
  int rc = elementwise::gate_check(f);
  if (rc) return rc;
  if (!workspace || workspace_bytes < elementwise::gate_bwd_workspace_bytes(*p)) return TOPS_E_WORKSPACE;
  return elementwise::gate_bwd(*p, workspace, (cudaStream_t)stream);
}

extern "C" int tops_b200_l2norm_fwd(const tops_norm_params* p, void* stream) {
  if (!p) return TOPS_E_NULL;
  if (!valid_dtype(p->dtype)) return TOPS_E_BAD_DTYPE;
  int rc = elementwise::norm_check(*p);
  return rc ? rc : elementwise::l2norm_fwd(*p, (cudaStream_t)stream);
}

extern "C" int tops_b200_l2norm_bwd(const tops_norm_params* p, void* stream) {
  if (!p) return TOPS_E_NULL;
  if (!valid_dtype(p->dtype)) return TOPS_E_BAD_DTYPE;
  tops_norm_params q = *p;
  q.y = q.dx;
  int rc = elementwise::norm_check(q);
  return rc ? rc : elementwise::l2norm_bwd(*p, (cudaStream_t)stream);
}

extern "C" int tops_b200_rmsnorm_gated_fwd(const tops_norm_params* p, void* stream) {
  if (!p) return TOPS_E_NULL;
  if (!valid_dtype(p->dtype)) return TOPS_E_BAD_DTYPE;
  int rc = elementwise::norm_check(*p);
  return rc ? rc : elementwise::rmsnorm_gated_fwd(*p, (cudaStream_t)stream);
}

extern "C" size_t tops_b200_rmsnorm_gated_bwd_workspace_bytes(const tops_norm_params* p) {
  if (!p || p->rows < 1 || p->D < 1) return 0;
  return elementwise::rmsnorm_gated_bwd_workspace_bytes(*p);
}

extern "C" int tops_b200_rmsnorm_gated_bwd(const tops_norm_params* p, void* workspace, size_t workspace_bytes,
                                           void* stream) {
  if (!p) return TOPS_E_NULL;
  if (!valid_dtype(p->dtype)) return TOPS_E_BAD_DTYPE;
  tops_norm_params q = *p;
  q.y = q.dx;
  int rc = elementwise::norm_check(q);
  if (rc) return rc;
  if (!workspace || workspace_bytes < elementwise::rmsnorm_gated_bwd_workspace_bytes(*p)) return TOPS_E_WORKSPACE;
  return elementwise::rmsnorm_gated_bwd(*p, workspace, (cudaStream_t)stream);
}

// ---- state exchange of a time-sharded sequence -------------------------------------
extern "C" size_t tops_b200_chunk_state_exchange_pack_workspace_bytes(const tops_state_pack_params* p) {
  if (!p || check_problem(p->pb) || !sm100::supported(p->pb)) return 0;
  return sm100::summary_workspace_bytes(p->pb);
}

extern "C" int tops_b200_chunk_state_exchange_pack(const tops_state_pack_params* p, void* workspace, size_t workspace_bytes,
                                                   void* stream) {
  if (!p || !p->x || !p->g || !p->y || !p->state_out) return TOPS_E_NULL;
  int rc = check_problem(p->pb);
  if (rc) return rc;
  if (!sm100::supported(p->pb)) return TOPS_E_UNSUPPORTED;
  if (!workspace || workspace_bytes < sm100::summary_workspace_bytes(p->pb)) return TOPS_E_WORKSPACE;
  return sm100::state_summary(p->pb, p->reverse != 0, p->x, p->g, p->y, p->state_out, workspace, (cudaStream_t)stream);
}

extern "C" int tops_b200_chunk_state_exchange_apply(const tops_state_apply_params* p, void* stream) {
  if (!p || !p->P || !p->S || !p->out_in) return TOPS_E_NULL;
  if (p->R < 1 || p->rank < 0 || p->rank >= p->R || p->BH < 1 || p->K < 1 || p->V < 1 || (p->V % 4) != 0)
    return TOPS_E_BAD_SHAPE;
  const void* ptrs[] = {p->first, p->P, p->S, p->out_in, p->out_all};
  for (const void* x : ptrs)
    if (reinterpret_cast<uintptr_t>(x) & 15) return TOPS_E_ALIGN;
  return generic::launch_fold_shards(p->first, p->P, p->S, p->out_in, p->out_all, p->R, p->rank, p->reverse,
                                     (size_t)p->BH, p->K, p->V, (cudaStream_t)stream);
}
