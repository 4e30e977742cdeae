/* Stand-in for the CUDA driver's virtual-memory and multicast entry points, for tests on machines without a GPU.
 * "Device memory" is a memfd; a shareable handle is a duplicate of that descriptor; mapping is mmap.  It keeps
 * enough book-keeping (live handles, bindings, mappings) for a test to see what the code under test released.
 * A fabric handle (type 8) is 64 bytes naming the slot; importing one works in the process that made it and in its forked
 * children, which is what a test needs.  FAKE_CUDA_NO_FABRIC=1 makes allocations that ask for fabric handles fail, as a
 * machine without an IMEX channel does.
 * Only what csrc/mem/cuda_device.cc resolves by name is here. */
#define _GNU_SOURCE
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

typedef int CUresult;
typedef int CUdevice;
typedef unsigned long long CUdeviceptr;
typedef unsigned long long Handle;

#define MAXH 256
static struct { int fd; size_t size; int live; int is_mc; int bound; int devices; } g_h[MAXH];
static int g_maps = 0;
static int g_fabric_exports = 0, g_fabric_imports = 0;
#define TYPE_FABRIC 8

static int slot_new(void) {
  for (int i = 1; i < MAXH; ++i)
    if (!g_h[i].live) { memset(&g_h[i], 0, sizeof(g_h[i])); g_h[i].live = 1; return i; }
  return 0;
}

CUresult cuGetErrorString(CUresult e, const char** s) { *s = e == 0 ? "no error" : "stand-in driver error"; return 0; }
CUresult cuCtxGetDevice(CUdevice* d) { *d = 0; return 0; }
CUresult cuDeviceGetAttribute(int* v, int attr, CUdevice d) { (void)attr; (void)d; *v = 1; return 0; }
CUresult cuMemGetAllocationGranularity(size_t* g, const void* prop, int flags) { (void)prop; (void)flags; *g = 2u << 20; return 0; }

CUresult cuMemCreate(Handle* h, size_t size, const void* prop, unsigned long long flags) {
  (void)flags;
  /* CUmemAllocationProp starts with { int type; int requestedHandleTypes; ... } */
  if (prop && (((const int*)prop)[1] & TYPE_FABRIC) && getenv("FAKE_CUDA_NO_FABRIC")) return 801;
  int i = slot_new();
  if (!i) return 2;
  g_h[i].fd = memfd_create("fake-cuda", MFD_CLOEXEC);
  if (g_h[i].fd < 0 || ftruncate(g_h[i].fd, (off_t)size) != 0) { g_h[i].live = 0; return 2; }
  g_h[i].size = size;
  *h = (Handle)i;
  return 0;
}
CUresult cuMemRelease(Handle h) {
  if (h == 0 || h >= MAXH || !g_h[h].live) return 1;
  close(g_h[h].fd);
  g_h[h].live = 0;
  return 0;
}
CUresult cuMemAddressReserve(CUdeviceptr* p, size_t size, size_t align, CUdeviceptr addr, unsigned long long flags) {
  (void)align; (void)addr; (void)flags;
  void* v = mmap(NULL, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (v == MAP_FAILED) return 2;
  *p = (CUdeviceptr)(uintptr_t)v;
  return 0;
}
CUresult cuMemAddressFree(CUdeviceptr p, size_t size) { return munmap((void*)(uintptr_t)p, size) == 0 ? 0 : 1; }
CUresult cuMemMap(CUdeviceptr p, size_t size, size_t off, Handle h, unsigned long long flags) {
  (void)flags;
  if (h == 0 || h >= MAXH || !g_h[h].live) return 1;
  void* v = mmap((void*)(uintptr_t)p, size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, g_h[h].fd, (off_t)off);
  if (v == MAP_FAILED) return 2;
  ++g_maps;
  return 0;
}
CUresult cuMemUnmap(CUdeviceptr p, size_t size) {
  void* v = mmap((void*)(uintptr_t)p, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED | MAP_NORESERVE, -1, 0);
  if (v == MAP_FAILED) return 1;
  --g_maps;
  return 0;
}
CUresult cuMemSetAccess(CUdeviceptr p, size_t size, const void* desc, size_t n) { (void)p; (void)size; (void)desc; (void)n; return 0; }
CUresult cuMemExportToShareableHandle(void* out, Handle h, int type, unsigned long long flags) {
  (void)flags;
  if (h == 0 || h >= MAXH || !g_h[h].live) return 1;
  if (type == TYPE_FABRIC) {
    memset(out, 0, 64);
    memcpy(out, "FAKEFABR", 8);
    memcpy((char*)out + 8, &h, sizeof(h));
    ++g_fabric_exports;
    return 0;
  }
  int fd = dup(g_h[h].fd);
  if (fd < 0) return 2;
  *(int*)out = fd;
  return 0;
}
CUresult cuMemImportFromShareableHandle(Handle* h, void* os_handle, int type) {
  if (type == TYPE_FABRIC) {
    Handle src = 0;
    if (memcmp(os_handle, "FAKEFABR", 8) != 0) return 1;
    memcpy(&src, (const char*)os_handle + 8, sizeof(src));
    if (src == 0 || src >= MAXH || !g_h[src].live) return 1;
    int j = slot_new();
    if (!j) return 2;
    g_h[j].fd = dup(g_h[src].fd);
    g_h[j].size = g_h[src].size;
    *h = (Handle)j;
    ++g_fabric_imports;
    return 0;
  }
  int fd = (int)(intptr_t)os_handle;
  struct stat st;
  if (fstat(fd, &st) != 0) return 1;
  int i = slot_new();
  if (!i) return 2;
  g_h[i].fd = dup(fd);
  g_h[i].size = (size_t)st.st_size;
  *h = (Handle)i;
  return 0;
}

struct McProp { unsigned int numDevices; size_t size; unsigned long long handleTypes; unsigned long long flags; };
CUresult cuMulticastGetGranularity(size_t* g, const struct McProp* p, int which) { (void)p; (void)which; *g = 2u << 20; return 0; }
CUresult cuMulticastCreate(Handle* h, const struct McProp* p) {
  CUresult r = cuMemCreate(h, p->size, NULL, 0);
  if (r == 0) g_h[*h].is_mc = 1;
  return r;
}
CUresult cuMulticastAddDevice(Handle h, CUdevice d) {
  (void)d;
  if (h == 0 || h >= MAXH || !g_h[h].live) return 1;
  g_h[h].devices++;
  return 0;
}
CUresult cuMulticastBindMem(Handle mc, size_t mc_off, Handle mem, size_t mem_off, size_t size, unsigned long long flags) {
  (void)mc_off; (void)mem_off; (void)size; (void)flags;
  if (mc == 0 || mc >= MAXH || !g_h[mc].live || mem == 0 || mem >= MAXH || !g_h[mem].live) return 1;
  g_h[mc].bound++;
  return 0;
}
CUresult cuMulticastUnbind(Handle mc, CUdevice d, size_t off, size_t size) {
  (void)d; (void)off; (void)size;
  if (mc == 0 || mc >= MAXH || !g_h[mc].live || g_h[mc].bound <= 0) return 1;
  g_h[mc].bound--;
  return 0;
}

/* ---- what the tests look at ---- */
int fake_cuda_handle_alive(Handle h) { return h > 0 && h < MAXH && g_h[h].live; }
int fake_cuda_handle_bound(Handle h) { return h > 0 && h < MAXH && g_h[h].live ? g_h[h].bound : -1; }
int fake_cuda_live_handles(void) { int n = 0; for (int i = 1; i < MAXH; ++i) n += g_h[i].live; return n; }
int fake_cuda_mappings(void) { return g_maps; }
int fake_cuda_fabric_exports(void) { return g_fabric_exports; }
int fake_cuda_fabric_imports(void) { return g_fabric_imports; }
