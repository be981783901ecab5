// NUMA placement of the host mirrors and of the correction workers.
//
// On a two-socket host every GPU hangs off one socket.  The host correction gathers 256-byte
// rows at random from a mirror of many gigabytes; with the mirror on the other socket, or the
// workers there, every row crosses the socket interconnect.  These entry points read the
// machine's layout from sysfs, bind a range of host memory to one node (mbind, best before the
// memory is first touched) and restrict the correction workers to one node's processors.  The
// reference leaves placement to the operating system's first-touch policy; there is no
// counterpart to cite.
//
// The sysfs tree is read below $JF_SYSFS_ROOT when that is set (tests point it at a made-up
// tree), else below /sys.
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "../../include/jetfire_b200.h"
#include "numa_place.h"

namespace {

std::string sysfs_root() {
  const char* r = std::getenv("JF_SYSFS_ROOT");
  return (r && *r) ? std::string(r) : std::string("/sys");
}

bool read_line(const std::string& path, std::string* out) {
  FILE* f = std::fopen(path.c_str(), "r");
  if (!f) return false;
  char buf[4096];
  const bool ok = std::fgets(buf, sizeof buf, f) != nullptr;
  std::fclose(f);
  if (!ok) return false;
  out->assign(buf);
  while (!out->empty() && (out->back() == '\n' || out->back() == ' ' || out->back() == '\r')) out->pop_back();
  return true;
}

// "0-3,8,10-11" -> {0,1,2,3,8,10,11}; false on anything else
bool parse_list(const std::string& s, std::vector<int>* out) {
  out->clear();
  size_t i = 0;
  while (i < s.size()) {
    char* end = nullptr;
    errno = 0;
    const long a = std::strtol(s.c_str() + i, &end, 10);
    if (end == s.c_str() + i || errno || a < 0 || a > (1 << 20)) return false;
    long b = a;
    i = static_cast<size_t>(end - s.c_str());
    if (i < s.size() && s[i] == '-') {
      ++i;
      b = std::strtol(s.c_str() + i, &end, 10);
      if (end == s.c_str() + i || errno || b < a || b > (1 << 20)) return false;
      i = static_cast<size_t>(end - s.c_str());
    }
    for (long v = a; v <= b; ++v) out->push_back(static_cast<int>(v));
    if (i < s.size()) {
      if (s[i] != ',') return false;
      ++i;
    }
  }
  return true;
}

bool online_nodes(std::vector<int>* nodes) {
  std::string line;
  if (!read_line(sysfs_root() + "/devices/system/node/online", &line)) return false;
  return parse_list(line, nodes) && !nodes->empty();
}

std::atomic<int> g_worker_node{-1};

}  // namespace

namespace jf {

bool node_cpus(int node, std::vector<int>* cpus) {
  std::string line;
  if (node < 0 || !read_line(sysfs_root() + "/devices/system/node/node" + std::to_string(node) + "/cpulist", &line))
    return false;
  return parse_list(line, cpus) && !cpus->empty();
}

int worker_node() { return g_worker_node.load(std::memory_order_relaxed); }

// Restricts the calling thread to the processors of `node`; false (affinity untouched) when the
// node is unknown or the system refuses.
bool pin_this_thread_to_node(int node) {
  std::vector<int> cpus;
  if (!node_cpus(node, &cpus)) return false;
  cpu_set_t set;
  CPU_ZERO(&set);
  int n = 0;
  for (int c : cpus)
    if (c < CPU_SETSIZE) { CPU_SET(c, &set); ++n; }
  return n > 0 && sched_setaffinity(0, sizeof set, &set) == 0;
}

}  // namespace jf

// Memory nodes the system reports online; 1 when it reports nothing (no sysfs, not Linux).
extern "C" int32_t jf_numa_node_count(void) {
  std::vector<int> nodes;
  return online_nodes(&nodes) ? static_cast<int32_t>(nodes.size()) : 1;
}

// Node the GPU's PCI function is attached to; -1 when the system does not say (single-node
// machines and virtual machines usually report -1).
extern "C" int32_t jf_numa_node_of_device(int32_t device) {
  char bus[32] = {0};
  if (cudaDeviceGetPCIBusId(bus, sizeof bus, device) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  for (char* p = bus; *p; ++p)
    if (*p >= 'A' && *p <= 'F') *p = static_cast<char>(*p - 'A' + 'a');   // sysfs names are lower case
  std::string line;
  if (!read_line(sysfs_root() + "/bus/pci/devices/" + bus + "/numa_node", &line)) return -1;
  char* end = nullptr;
  const long v = std::strtol(line.c_str(), &end, 10);
  return (end == line.c_str() || v < 0) ? -1 : static_cast<int32_t>(v);
}

// The processors of a node, ascending.  *count receives how many there are (also when more than
// `capacity`, in which case only the first `capacity` are written).
extern "C" jf_status_t jf_numa_node_cpus(int32_t node, int32_t* cpus, int32_t capacity, int32_t* count) {
  if (!count || capacity < 0 || (capacity > 0 && !cpus)) return JF_ERR_ARG;
  std::vector<int> list;
  if (!jf::node_cpus(node, &list)) return JF_ERR_UNSUPPORTED;
  *count = static_cast<int32_t>(list.size());
  for (int i = 0; i < capacity && i < static_cast<int>(list.size()); ++i) cpus[i] = list[i];
  return JF_OK;
}

// Binds the whole pages inside [ptr, ptr + bytes) to `node` (mbind, MPOL_BIND; pages already
// present are moved).  Pinned pages cannot move: bind before the memory is registered with the
// driver.  JF_ERR_UNSUPPORTED when the node is not online or the system refuses.
extern "C" jf_status_t jf_bind_memory_to_node(void* ptr, uint64_t bytes, int32_t node) {
  if (!ptr || bytes == 0 || node < 0 || node >= 1024) return JF_ERR_ARG;
  std::vector<int> nodes;
  if (!online_nodes(&nodes)) return JF_ERR_UNSUPPORTED;
  bool present = false;
  for (int n : nodes) present |= (n == node);
  if (!present) return JF_ERR_UNSUPPORTED;
  const long page = sysconf(_SC_PAGESIZE);
  if (page <= 0) return JF_ERR_UNSUPPORTED;
  const uintptr_t pg = static_cast<uintptr_t>(page);
  const uintptr_t lo = (reinterpret_cast<uintptr_t>(ptr) + pg - 1) & ~(pg - 1);
  const uintptr_t hi = (reinterpret_cast<uintptr_t>(ptr) + bytes) & ~(pg - 1);
  if (hi <= lo) return JF_OK;
#ifdef SYS_mbind
  constexpr int kBind = 2;        // MPOL_BIND
  constexpr unsigned kMove = 2;   // MPOL_MF_MOVE
  unsigned long mask[1024 / (8 * sizeof(unsigned long))] = {0};
  mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
  const long rc = syscall(SYS_mbind, reinterpret_cast<void*>(lo), static_cast<unsigned long>(hi - lo), kBind, mask,
                          static_cast<unsigned long>(1024 + 1), kMove);
  return rc == 0 ? JF_OK : JF_ERR_UNSUPPORTED;
#else
  return JF_ERR_UNSUPPORTED;
#endif
}

// Correction workers started from now on run only on the processors of `node` (-1: anywhere).
// A running pool is restarted by the next job.  JF_ERR_UNSUPPORTED for a node without
// processors.
extern "C" jf_status_t jf_set_cpu_attn_node(int32_t node) {
  if (node < -1) return JF_ERR_ARG;
  if (node >= 0) {
    std::vector<int> cpus;
    if (!jf::node_cpus(node, &cpus)) return JF_ERR_UNSUPPORTED;
  }
  g_worker_node.store(node, std::memory_order_relaxed);
  return JF_OK;
}

extern "C" int32_t jf_get_cpu_attn_node(void) { return jf::worker_node(); }
