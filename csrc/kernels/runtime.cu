// Runtime state of the kernel library, one set per CUDA device: the status word that
// bounded waits report into (plus the wait limit they read), the E8P decode tables, the
// start-up workspaces, and the driver entry point used to encode TMA tensor maps.  Every
// accessor answers for the device that is current on the calling thread, so a process that
// drives several GPUs gets separate state on each.
#include <cuda.h>
#include <atomic>
#include <mutex>

#include "api.h"
#include "common.cuh"
#include "e8p_basis.h"
#include "tma.h"

namespace orinfer {

namespace {
constexpr int MAX_DEVICES = 64;
constexpr int MAX_SLOTS = 256;

struct DeviceState {
  bool ready = false;
  int* status = nullptr;          // int32 [4]: status, -, wait limit / 1024 cycles, -
  E8pTables* tables = nullptr;
  int* splitk = nullptr;
  int* splitk_tickets = nullptr;  // int32 [SPLITK_TICKETS], zero between launches
  int* gemv_ws = nullptr;
  bool used[MAX_SLOTS] = {};
};

std::mutex g_mutex;
DeviceState g_dev[MAX_DEVICES];
PFN_encodeTiled g_encode = nullptr;
std::atomic<int> g_slots{0};

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
  return dev;
}

// Position of coordinate c's 4-bit field inside a table word.
int field_of(int c) { return c < 4 ? 2 * c : 2 * (c - 4) + 1; }

void build_tables(E8pTables* host) {
  static const int coord_bit[8] = {0, 4, 1, 5, 2, 6, 3, 7};
  int8_t basis[256][8];
  build_e8p_basis(basis);
  for (int i = 0; i < 256; ++i) {
    uint32_t e = 0, s = 0;
    const int par = __builtin_popcount(i) & 1;
    const int flips = i ^ par;
    for (int c = 0; c < 8; ++c) {
      const uint32_t u = static_cast<uint32_t>((basis[i][c] + 14) / 4);       // 1..6
      e |= (2u * u) << (4 * field_of(c));
      const uint32_t f = (flips >> coord_bit[c]) & 1;
      s |= ((f ? 0xEu : 0u) | static_cast<uint32_t>(1 - par)) << (4 * field_of(c));
    }
    host->e2[i] = e;
    host->sg[i] = s;
  }
}
}  // namespace

cudaError_t runtime_ensure_init() {
  const int dev = current_device();
  if (dev < 0) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& d = g_dev[dev];
  if (d.ready) return cudaSuccess;
  static E8pTables host;
  build_tables(&host);
  cudaError_t e = cudaMalloc(&d.status, 4 * sizeof(int));
  if (e != cudaSuccess) return e;
  const int init[4] = {0, 0, static_cast<int>(WAIT_LIMIT_CYCLES >> 10), 0};
  e = cudaMemcpy(d.status, init, sizeof(init), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&d.tables, sizeof(E8pTables));
  if (e != cudaSuccess) return e;
  e = cudaMemcpy(d.tables, &host, sizeof(E8pTables), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&d.splitk, SPLITK_WORKSPACE_BYTES);
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&d.splitk_tickets, SPLITK_TICKETS * sizeof(int));
  if (e != cudaSuccess) return e;
  e = cudaMemset(d.splitk_tickets, 0, SPLITK_TICKETS * sizeof(int));
  if (e != cudaSuccess) return e;
  const size_t ws = (static_cast<size_t>(8) * GEMV_WS_COLS + GEMV_WS_TICKETS) * sizeof(int);
  e = cudaMalloc(&d.gemv_ws, ws);
  if (e != cudaSuccess) return e;
  e = cudaMemset(d.gemv_ws, 0, ws);
  if (e != cudaSuccess) return e;
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess) return e;
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return cudaErrorNotSupported;
    g_encode = reinterpret_cast<PFN_encodeTiled>(fn);
  }
  d.ready = true;
  return cudaSuccess;
}

namespace {
DeviceState* ready_state() {
  const int dev = current_device();
  if (dev < 0 || !g_dev[dev].ready) return nullptr;
  return &g_dev[dev];
}
}  // namespace

int* runtime_status_ptr() {
  DeviceState* d = ready_state();
  return d ? d->status : nullptr;
}
int* runtime_splitk_workspace() {
  DeviceState* d = ready_state();
  return d ? d->splitk : nullptr;
}
int* runtime_splitk_tickets() {
  DeviceState* d = ready_state();
  return d ? d->splitk_tickets : nullptr;
}
int* runtime_gemv_workspace() {
  DeviceState* d = ready_state();
  return d ? d->gemv_ws : nullptr;
}
const E8pTables* runtime_e8p_tables() {
  DeviceState* d = ready_state();
  return d ? d->tables : nullptr;
}
PFN_encodeTiled runtime_tma_encoder() { return g_encode; }

int runtime_new_slot() {
  const int s = g_slots.fetch_add(1);
  return s < MAX_SLOTS ? s : -1;
}

bool runtime_first_use(int slot) {
  const int dev = current_device();
  if (dev < 0 || slot < 0 || slot >= MAX_SLOTS) return true;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_dev[dev].used[slot]) return false;
  g_dev[dev].used[slot] = true;
  return true;
}

}  // namespace orinfer

extern "C" {

int orinfer_init(void) { return static_cast<int>(orinfer::runtime_ensure_init()); }

int orinfer_read_status(int* out4) {
  if (orinfer::runtime_ensure_init() != cudaSuccess) return -2;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemcpy(out4, orinfer::runtime_status_ptr(), 4 * sizeof(int),
                                     cudaMemcpyDeviceToHost));
}

// Copies the four status ints to (pinned) host memory behind the work already queued on
// `stream`; no synchronisation.  The caller reads them after its own wait on that stream.
int orinfer_status_async(int* host_out4, cudaStream_t stream) {
  if (orinfer::runtime_ensure_init() != cudaSuccess) return -2;
  return static_cast<int>(cudaMemcpyAsync(host_out4, orinfer::runtime_status_ptr(),
                                          4 * sizeof(int), cudaMemcpyDeviceToHost, stream));
}

int orinfer_clear_status(void) {
  if (orinfer::runtime_ensure_init() != cudaSuccess) return -2;
  return static_cast<int>(cudaMemset(orinfer::runtime_status_ptr(), 0, sizeof(int)));
}

// How long a bounded device wait spins before it gives up, in microseconds of a ~2 GHz clock.
int orinfer_set_wait_limit_us(long long us) {
  if (us < 1 || us > 60000000LL) return -1;
  if (orinfer::runtime_ensure_init() != cudaSuccess) return -2;
  const int k = static_cast<int>((us * 2000LL) >> 10) + 1;
  return static_cast<int>(cudaMemcpy(orinfer::runtime_status_ptr() + orinfer::STATUS_LIMIT_WORD,
                                     &k, sizeof(int), cudaMemcpyHostToDevice));
}

// Ordinal of the device whose runtime state the calling thread would use, or -1.
int orinfer_current_device(void) { return orinfer::current_device(); }

const void* orinfer_e8p_tables_device(void) {
  if (orinfer::runtime_ensure_init() != cudaSuccess) return nullptr;
  return orinfer::runtime_e8p_tables();
}

int orinfer_e8p_basis_host(int8_t* out) {
  int8_t b[256][8];
  orinfer::build_e8p_basis(b);
  for (int i = 0; i < 256; ++i)
    for (int d = 0; d < 8; ++d) out[i * 8 + d] = b[i][d];
  return 0;
}

}  // extern "C"
