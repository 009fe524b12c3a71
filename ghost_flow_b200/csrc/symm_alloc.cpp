// Symmetric (peer-mapped) memory without a tensor library: one physical allocation per rank, every rank's
// allocation mapped into every process at base + rank * size.
//
// The flow is the CUDA virtual-memory-management one: cuMemCreate (shareable as a POSIX file descriptor) ->
// cuMemExportToShareableHandle -> the descriptors travel between the processes of one node over unix-domain sockets
// (SCM_RIGHTS) -> cuMemImportFromShareableHandle -> cuMemAddressReserve for world * size bytes -> cuMemMap of every
// rank's handle at its slot -> cuMemSetAccess for the local device. Kernels then address a peer's buffer as
// base + peer * size + offset; no library sits between the kernel and NVLink.
//
// The driver is reached through a table of function pointers filled with dlopen("libcuda.so.1"), so this file has no
// link-time dependency on CUDA. The same table can be pointed at a host stand-in (gf_symm_use_host_driver) in which
// "device memory" is a memfd, export is dup(), the address reservation is an inaccessible anonymous mapping and
// cuMemMap is a MAP_FIXED shared mapping: the whole flow, descriptor passing between processes included, then runs
// and can be tested on a machine without a GPU, and what a rank writes into its slot is really visible to its peers.
//
// Status: exercised with the host stand-in (tests/test_symm_alloc_cpu.py). Not run on a GPU; the package keeps using
// torch.distributed._symmetric_memory unless GF_SYMM_ALLOC=own is set. In-switch multicast objects
// (cuMulticastCreate / cuMulticastBindMem) are not covered.
// The reference has one process and one Vec<u8> pool (ghostflow-cuda/src/memory.rs); nothing there is shared.
#include <dlfcn.h>
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

#ifdef GF_HAVE_CUDA_H
#include <cuda.h>      // only to check the hand-written ABI below against the toolkit's header; nothing is linked
#endif

#define GF_API extern "C" __attribute__((visibility("default")))

namespace {

// ---- the part of the driver API that is used, with the driver's own ABI (values from cuda.h, CUDA 12)
typedef unsigned long long CUdeviceptr_t;
typedef unsigned long long CUmemHandle_t;
struct MemLocation { int type; int id; };                                    // CUmemLocation
struct MemAllocationProp {                                                    // CUmemAllocationProp
  int type; int requestedHandleTypes; MemLocation location; void* win32HandleMetaData;
  struct { unsigned char compressionType, gpuDirectRDMACapable; unsigned short usage; unsigned char reserved[4]; } allocFlags;
};
struct MemAccessDesc { MemLocation location; int flags; };                    // CUmemAccessDesc
constexpr int kAllocTypePinned = 1, kLocationDevice = 1, kHandlePosixFd = 1, kAccessReadWrite = 3, kGranMinimum = 0;

#ifdef GF_HAVE_CUDA_H
static_assert(sizeof(MemAllocationProp) == sizeof(CUmemAllocationProp), "CUmemAllocationProp layout");
static_assert(sizeof(MemAccessDesc) == sizeof(CUmemAccessDesc), "CUmemAccessDesc layout");
static_assert(sizeof(MemLocation) == sizeof(CUmemLocation), "CUmemLocation layout");
static_assert(kAllocTypePinned == CU_MEM_ALLOCATION_TYPE_PINNED && kLocationDevice == CU_MEM_LOCATION_TYPE_DEVICE &&
              kHandlePosixFd == CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR &&
              kAccessReadWrite == CU_MEM_ACCESS_FLAGS_PROT_READWRITE && kGranMinimum == CU_MEM_ALLOC_GRANULARITY_MINIMUM,
              "driver enum values");
static_assert(sizeof(CUdeviceptr_t) == sizeof(CUdeviceptr) && sizeof(CUmemHandle_t) == sizeof(CUmemGenericAllocationHandle),
              "handle widths");
#endif

struct DriverApi {
  int (*init)(unsigned);
  int (*get_granularity)(size_t*, const MemAllocationProp*, int);
  int (*create)(CUmemHandle_t*, size_t, const MemAllocationProp*, unsigned long long);
  int (*export_handle)(void*, CUmemHandle_t, int, unsigned long long);
  int (*import_handle)(CUmemHandle_t*, void*, int);
  int (*address_reserve)(CUdeviceptr_t*, size_t, size_t, CUdeviceptr_t, unsigned long long);
  int (*map)(CUdeviceptr_t, size_t, size_t, CUmemHandle_t, unsigned long long);
  int (*set_access)(CUdeviceptr_t, size_t, const MemAccessDesc*, size_t);
  int (*unmap)(CUdeviceptr_t, size_t);
  int (*release)(CUmemHandle_t);
  int (*address_free)(CUdeviceptr_t, size_t);
};

// ---- host stand-in: memfd-backed "allocations"
int h_init(unsigned) { return 0; }
int h_gran(size_t* g, const MemAllocationProp*, int) { *g = (size_t)sysconf(_SC_PAGESIZE); return 0; }
int h_create(CUmemHandle_t* h, size_t size, const MemAllocationProp*, unsigned long long) {
  int fd = memfd_create("gf_symm", 0);
  if (fd < 0 || ftruncate(fd, (off_t)size) != 0) return 2;
  *h = (CUmemHandle_t)fd;
  return 0;
}
int h_export(void* out, CUmemHandle_t h, int, unsigned long long) {
  int fd = dup((int)h);
  if (fd < 0) return 1;
  *(int*)out = fd;
  return 0;
}
int h_import(CUmemHandle_t* h, void* os_handle, int) { *h = (CUmemHandle_t)(intptr_t)os_handle; return 0; }
int h_reserve(CUdeviceptr_t* p, size_t size, size_t, CUdeviceptr_t, unsigned long long) {
  void* a = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (a == MAP_FAILED) return 2;
  *p = (CUdeviceptr_t)(uintptr_t)a;
  return 0;
}
int h_map(CUdeviceptr_t p, size_t size, size_t offset, CUmemHandle_t h, unsigned long long) {
  void* a = mmap((void*)(uintptr_t)p, size, PROT_NONE, MAP_SHARED | MAP_FIXED, (int)h, (off_t)offset);
  return a == MAP_FAILED ? 1 : 0;
}
int h_access(CUdeviceptr_t p, size_t size, const MemAccessDesc*, size_t) {
  return mprotect((void*)(uintptr_t)p, size, PROT_READ | PROT_WRITE) == 0 ? 0 : 1;
}
int h_unmap(CUdeviceptr_t p, size_t size) {
  void* a = mmap((void*)(uintptr_t)p, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED | MAP_NORESERVE, -1, 0);
  return a == MAP_FAILED ? 1 : 0;
}
int h_release(CUmemHandle_t h) { return close((int)h) == 0 ? 0 : 1; }
int h_free(CUdeviceptr_t p, size_t size) { return munmap((void*)(uintptr_t)p, size) == 0 ? 0 : 1; }

const DriverApi kHostDriver = {h_init, h_gran, h_create, h_export, h_import, h_reserve, h_map, h_access, h_unmap, h_release, h_free};
DriverApi g_cuda = {};
const DriverApi* g_api = nullptr;
bool g_host = false;
std::string g_error;

bool load_cuda() {
  if (g_cuda.create) return true;
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) { g_error = "libcuda.so.1 not found"; return false; }
  auto sym = [&](const char* n) { return dlsym(lib, n); };
  g_cuda.init = (int (*)(unsigned))sym("cuInit");
  g_cuda.get_granularity = (decltype(g_cuda.get_granularity))sym("cuMemGetAllocationGranularity");
  g_cuda.create = (decltype(g_cuda.create))sym("cuMemCreate");
  g_cuda.export_handle = (decltype(g_cuda.export_handle))sym("cuMemExportToShareableHandle");
  g_cuda.import_handle = (decltype(g_cuda.import_handle))sym("cuMemImportFromShareableHandle");
  g_cuda.address_reserve = (decltype(g_cuda.address_reserve))sym("cuMemAddressReserve");
  g_cuda.map = (decltype(g_cuda.map))sym("cuMemMap");
  g_cuda.set_access = (decltype(g_cuda.set_access))sym("cuMemSetAccess");
  g_cuda.unmap = (decltype(g_cuda.unmap))sym("cuMemUnmap");
  g_cuda.release = (decltype(g_cuda.release))sym("cuMemRelease");
  g_cuda.address_free = (decltype(g_cuda.address_free))sym("cuMemAddressFree");
  if (!g_cuda.init || !g_cuda.create || !g_cuda.export_handle || !g_cuda.import_handle || !g_cuda.address_reserve ||
      !g_cuda.map || !g_cuda.set_access || !g_cuda.unmap || !g_cuda.release || !g_cuda.address_free ||
      !g_cuda.get_granularity) {
    g_error = "the driver lacks the virtual-memory-management entry points";
    g_cuda = {};
    return false;
  }
  return true;
}

// ---- descriptor exchange between the ranks of one node
std::string sock_path(const std::string& dir, const std::string& job, int rank) {
  return dir + "/gfsymm_" + job + "_" + std::to_string(rank) + ".sock";
}

int send_fd(int sock, const sockaddr_un& to, int fd, int from_rank) {
  msghdr msg = {};
  iovec io = {&from_rank, sizeof(from_rank)};
  char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msg.msg_name = (void*)&to; msg.msg_namelen = sizeof(to);
  msg.msg_iov = &io; msg.msg_iovlen = 1;
  msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET; c->cmsg_type = SCM_RIGHTS; c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, 0) < 0 ? -1 : 0;
}

int recv_fd(int sock, int* from_rank) {
  msghdr msg = {};
  iovec io = {from_rank, sizeof(*from_rank)};
  char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msg.msg_iov = &io; msg.msg_iovlen = 1;
  msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, 0) < 0) return -1;
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_type != SCM_RIGHTS) return -1;
  int fd;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  return fd;
}

struct Symm {
  int rank = 0, world = 1;
  size_t size = 0;                 // bytes per rank, rounded to the granularity
  CUdeviceptr_t base = 0;
  std::vector<CUmemHandle_t> handles;
  std::vector<char> mapped;
  bool host = false;
};

}  // namespace

GF_API const char* gf_symm_last_error() { return g_error.c_str(); }

// 1: route every call to the host stand-in (memfd + mmap); 0: the CUDA driver.
GF_API int gf_symm_use_host_driver(int on) {
  g_host = on != 0;
  return 0;
}

// Collective over the `world` processes of one node. `sock_dir` must exist and be shared by them; `job` makes the
// socket names unique. On success *out is the allocation and every rank's slot is mapped and accessible.
GF_API int gf_symm_create(int device, size_t bytes, int rank, int world, const char* sock_dir, const char* job,
                          int timeout_s, void** out) {
  g_error.clear();
  if (!out || world < 1 || rank < 0 || rank >= world || bytes == 0 || !sock_dir || !job) { g_error = "bad argument"; return -1; }
  if (g_host) g_api = &kHostDriver;
  else { if (!load_cuda()) return -2; g_api = &g_cuda; }
  const DriverApi& d = *g_api;
  if (d.init(0) != 0) { g_error = "driver initialisation failed"; return -2; }
  MemAllocationProp prop = {};
  prop.type = kAllocTypePinned; prop.requestedHandleTypes = kHandlePosixFd;
  prop.location.type = kLocationDevice; prop.location.id = device;
  size_t gran = 0;
  if (d.get_granularity(&gran, &prop, kGranMinimum) != 0 || gran == 0) { g_error = "no allocation granularity"; return -3; }
  auto s = new Symm();
  s->rank = rank; s->world = world; s->host = g_host;
  s->size = (bytes + gran - 1) / gran * gran;
  s->handles.assign(world, 0);
  s->mapped.assign(world, 0);
  auto fail = [&](const char* what, int code) { g_error = what; delete s; return code; };
  if (d.create(&s->handles[rank], s->size, &prop, 0) != 0) return fail("cuMemCreate failed", -4);
  if (world > 1) {
    int my_fd = -1;
    if (d.export_handle(&my_fd, s->handles[rank], kHandlePosixFd, 0) != 0) return fail("export failed", -5);
    int sock = socket(AF_UNIX, SOCK_DGRAM, 0);
    sockaddr_un me = {};
    me.sun_family = AF_UNIX;
    const std::string mine = sock_path(sock_dir, job, rank);
    if (mine.size() >= sizeof(me.sun_path)) { close(sock); return fail("socket path too long", -6); }
    strcpy(me.sun_path, mine.c_str());
    unlink(mine.c_str());
    if (sock < 0 || bind(sock, (sockaddr*)&me, sizeof(me)) != 0) { if (sock >= 0) close(sock); return fail("cannot bind the exchange socket", -6); }
    timeval tv = {timeout_s > 0 ? timeout_s : 60, 0};
    setsockopt(sock, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    // send my descriptor to every peer (retry until the peer's socket exists), then collect world - 1 descriptors
    for (int p = 0; p < world; ++p) {
      if (p == rank) continue;
      sockaddr_un to = {};
      to.sun_family = AF_UNIX;
      strcpy(to.sun_path, sock_path(sock_dir, job, p).c_str());
      const time_t t0 = time(nullptr);
      while (send_fd(sock, to, my_fd, rank) != 0) {
        if (time(nullptr) - t0 > tv.tv_sec) { close(sock); unlink(mine.c_str()); return fail("a peer never opened its exchange socket", -7); }
        usleep(20000);
      }
    }
    for (int got = 0; got < world - 1; ++got) {
      int from = -1;
      const int fd = recv_fd(sock, &from);
      if (fd < 0 || from < 0 || from >= world || from == rank) { close(sock); unlink(mine.c_str()); return fail("descriptor exchange timed out", -7); }
      if (d.import_handle(&s->handles[from], (void*)(intptr_t)fd, kHandlePosixFd) != 0) { close(sock); unlink(mine.c_str()); return fail("import failed", -8); }
      if (!s->host) close(fd);        // the driver keeps its own reference; the stand-in's handle IS the descriptor
    }
    close(sock);
    unlink(mine.c_str());
    close(my_fd);
  }
  if (d.address_reserve(&s->base, s->size * world, gran, 0, 0) != 0) return fail("address reservation failed", -9);
  MemAccessDesc acc = {};
  acc.location.type = kLocationDevice; acc.location.id = device; acc.flags = kAccessReadWrite;
  for (int r = 0; r < world; ++r) {
    if (d.map(s->base + (CUdeviceptr_t)r * s->size, s->size, 0, s->handles[r], 0) != 0) return fail("cuMemMap failed", -10);
    s->mapped[r] = 1;
  }
  if (d.set_access(s->base, s->size * world, &acc, 1) != 0) return fail("cuMemSetAccess failed", -11);
  *out = s;
  return 0;
}

GF_API unsigned long long gf_symm_ptr(void* h, int rank) {
  auto s = (Symm*)h;
  return (s && rank >= 0 && rank < s->world) ? s->base + (CUdeviceptr_t)rank * s->size : 0;
}

GF_API unsigned long long gf_symm_bytes_per_rank(void* h) { return h ? ((Symm*)h)->size : 0; }

GF_API int gf_symm_destroy(void* h) {
  auto s = (Symm*)h;
  if (!s) return 0;
  const DriverApi& d = s->host ? kHostDriver : g_cuda;
  int rc = 0;
  for (int r = 0; r < s->world; ++r)
    if (s->mapped[r]) rc |= d.unmap(s->base + (CUdeviceptr_t)r * s->size, s->size);
  for (int r = 0; r < s->world; ++r)
    if (s->handles[r]) rc |= d.release(s->handles[r]);
  if (s->base) rc |= d.address_free(s->base, s->size * s->world);
  delete s;
  return rc ? -1 : 0;
}
