// Per-process runtime state of the kernel library: the device status word that
// bounded waits report into, the E8P decode tables in device memory, and the
// driver entry point used to encode TMA tensor maps.
#include <cuda.h>
#include <mutex>

#include "api.h"
#include "common.cuh"
#include "e8p_basis.h"
#include "tma.h"

namespace orinfer {

namespace {
std::mutex g_mutex;
bool g_ready = false;
int* g_status = nullptr;
E8pTables* g_tables = nullptr;
PFN_encodeTiled g_encode = nullptr;
int8_t g_basis[256][8];
int* g_splitk = nullptr;

uint32_t pack4(int a, int b, int c, int d) {
  return (static_cast<uint32_t>(a & 0xff)) | (static_cast<uint32_t>(b & 0xff) << 8) |
         (static_cast<uint32_t>(c & 0xff) << 16) | (static_cast<uint32_t>(d & 0xff) << 24);
}
}  // namespace

cudaError_t runtime_ensure_init() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_ready) return cudaSuccess;
  build_e8p_basis(g_basis);
  static E8pTables host;
  for (int i = 0; i < 256; ++i) {
    int pos[8];
    for (int d = 0; d < 8; ++d) pos[d] = g_basis[i][d] + 24;
    host.pos[i] = make_uint2(pack4(pos[0], pos[1], pos[2], pos[3]),
                             pack4(pos[4], pos[5], pos[6], pos[7]));
  }
  cudaError_t e = cudaMalloc(&g_status, 4 * sizeof(int));
  if (e != cudaSuccess) return e;
  e = cudaMemset(g_status, 0, 4 * sizeof(int));
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&g_tables, sizeof(E8pTables));
  if (e != cudaSuccess) return e;
  e = cudaMemcpy(g_tables, &host, sizeof(E8pTables), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&g_splitk, SPLITK_WORKSPACE_BYTES);
  if (e != cudaSuccess) return e;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return cudaErrorNotSupported;
  g_encode = reinterpret_cast<PFN_encodeTiled>(fn);
  g_ready = true;
  return cudaSuccess;
}

int* runtime_status_ptr() { return g_status; }
int* runtime_splitk_workspace() { return g_splitk; }
const E8pTables* runtime_e8p_tables() { return g_tables; }
PFN_encodeTiled runtime_tma_encoder() { return g_encode; }

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

int orinfer_clear_status(void) {
  if (orinfer::runtime_ensure_init() != cudaSuccess) return -2;
  return static_cast<int>(cudaMemset(orinfer::runtime_status_ptr(), 0, 4 * sizeof(int)));
}

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
