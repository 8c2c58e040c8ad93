// Collector of the debug build's device-side check records (see debug.cuh).
//
//   axb_debug_build()                  1 when the library was compiled with -DAXB_DEBUG, else 0
//   axb_debug_status(out4, file, n)    synchronises the current device, asks every translation unit for its
//                                      record and returns the first non-zero one: out4 = {code, source line,
//                                      value a, value b}, file = the unit's source file; 0 when all is clean.
//                                      The record that is returned is cleared.
#include "debug.cuh"
#include <cstring>

#ifdef AXB_DEBUG
namespace axb_dbg {
namespace {
constexpr int kMaxReaders = 64;
int (*g_readers[kMaxReaders])(int*);
const char* g_files[kMaxReaders];
int g_n = 0;
}  // namespace
void register_reader(int (*reader)(int*), const char* file) {
  if (g_n < kMaxReaders) {
    g_readers[g_n] = reader;
    g_files[g_n] = file;
    ++g_n;
  }
}
}  // namespace axb_dbg
#endif

extern "C" int axb_debug_build(void) {
#ifdef AXB_DEBUG
  return 1;
#else
  return 0;
#endif
}

extern "C" int axb_debug_status(int* out4, char* file, int file_len) {
  if (out4 != nullptr) out4[0] = out4[1] = out4[2] = out4[3] = 0;
  if (file != nullptr && file_len > 0) file[0] = 0;
#ifdef AXB_DEBUG
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  for (int i = 0; i < axb_dbg::g_n; ++i) {
    int rec[4] = {0, 0, 0, 0};
    if (axb_dbg::g_readers[i](rec) != 0) {
      if (out4 != nullptr) memcpy(out4, rec, sizeof(rec));
      if (file != nullptr && file_len > 0) {
        strncpy(file, axb_dbg::g_files[i], file_len - 1);
        file[file_len - 1] = 0;
      }
      return rec[0];
    }
  }
#endif
  return 0;
}
