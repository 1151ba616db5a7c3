// Token-shard data loader: raw uint16 token files (no header) are memory-mapped and walked with the
// same schedule as the reference DataLoaderLite (Data_Loader/dl_test.cpp:197-275): files whose name
// contains the split ("train"/"val") and ends in ".bin", sorted; position starts at B*T*rank and
// advances by B*T*world; the next shard is opened when fewer than B*T*world+1 tokens remain;
// skip_batches() fast-forwards for checkpoint resume.  Tokens are widened into caller-provided
// (pinned) int64 buffers so the host-to-device copy can be asynchronous.
#include <dirent.h>
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../kernels/host_utils.h"

using namespace cpb;

namespace {
struct Loader {
  std::vector<std::string> shards;
  int B = 0, T = 0, rank = 0, world = 1;
  size_t cur = 0, pos = 0;
  int fd = -1;
  void* map = nullptr;
  size_t bytes = 0, tokens = 0;

  void close_shard() {
    if (map) { munmap(map, bytes); map = nullptr; }
    if (fd >= 0) { ::close(fd); fd = -1; }
    bytes = tokens = 0;
  }
  int open_shard(size_t i) {
    close_shard();
    cur = i;
    fd = ::open(shards[i].c_str(), O_RDONLY);
    if (fd < 0) return set_error(CPB_ERR_ARG, "dataloader: cannot open %s", shards[i].c_str());
    struct stat st;
    if (fstat(fd, &st) != 0 || (st.st_size % 2)) return set_error(CPB_ERR_ARG, "dataloader: bad size of %s", shards[i].c_str());
    bytes = (size_t)st.st_size;
    tokens = bytes / 2;
    map = mmap(nullptr, bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) { map = nullptr; return set_error(CPB_ERR_ARG, "dataloader: mmap failed for %s", shards[i].c_str()); }
    madvise(map, bytes, MADV_SEQUENTIAL);
    pos = (size_t)B * T * rank;
    return CPB_OK;
  }
  int advance() { return open_shard((cur + 1) % shards.size()); }
  // Make sure one batch (B*T+1 tokens) starting at this rank's position lies inside the current shard, moving on
  // through at most every shard once.  A shard that is long enough for rank 0 may still be too short for a higher
  // rank's start offset B*T*rank, so the check runs after every open, not only once per loader.
  int ensure_batch() {
    const size_t need = (size_t)B * T + 1;
    for (size_t tries = 0; tries <= shards.size(); ++tries) {
      if (pos + need <= tokens) return CPB_OK;
      int rc = advance();
      if (rc) return rc;
    }
    return set_error(CPB_ERR_ARG, "dataloader: no shard holds a batch of %d x %d tokens at rank %d of %d", B, T, rank, world);
  }
};
}  // namespace

extern "C" int cpb_dl_open(const char* root, const char* split, int B, int T, int rank, int world, void** out) {
  DIR* d = opendir(root);
  if (!d) return set_error(CPB_ERR_ARG, "dataloader: cannot open directory %s", root);
  auto* L = new Loader();
  L->B = B; L->T = T; L->rank = rank; L->world = world;
  while (dirent* e = readdir(d)) {
    std::string n = e->d_name;
    if (n.size() > 4 && n.substr(n.size() - 4) == ".bin" && n.find(split) != std::string::npos)
      L->shards.push_back(std::string(root) + "/" + n);
  }
  closedir(d);
  std::sort(L->shards.begin(), L->shards.end());
  if (L->shards.empty()) { delete L; return set_error(CPB_ERR_ARG, "dataloader: no '%s' *.bin shard under %s", split, root); }
  int rc = L->open_shard(0);
  if (rc) { delete L; return rc; }
  *out = L;
  return CPB_OK;
}

extern "C" int cpb_dl_num_shards(void* h) { return (int)((Loader*)h)->shards.size(); }
extern "C" long cpb_dl_position(void* h) { return (long)((Loader*)h)->pos; }
extern "C" int cpb_dl_shard(void* h) { return (int)((Loader*)h)->cur; }

extern "C" int cpb_dl_next(void* h, int64_t* x, int64_t* y) {
  auto* L = (Loader*)h;
  const size_t BT = (size_t)L->B * L->T;
  { int rc = L->ensure_batch(); if (rc) return rc; }
  const uint16_t* t = (const uint16_t*)L->map + L->pos;
  for (size_t i = 0; i < BT; ++i) { x[i] = t[i]; y[i] = t[i + 1]; }
  L->pos += BT * (size_t)L->world;
  if (L->pos + BT * (size_t)L->world + 1 > L->tokens) { int rc = L->advance(); if (rc) return rc; }
  return CPB_OK;
}

extern "C" int cpb_dl_skip(void* h, long n) {
  auto* L = (Loader*)h;
  const size_t BT = (size_t)L->B * L->T, stride = BT * (size_t)L->world;
  for (long i = 0; i < n; ++i) {
    { int rc = L->ensure_batch(); if (rc) return rc; }
    L->pos += stride;
    if (L->pos + stride + 1 > L->tokens) { int rc = L->advance(); if (rc) return rc; }
  }
  return CPB_OK;
}

extern "C" int cpb_dl_reset(void* h) { return ((Loader*)h)->open_shard(0); }

extern "C" void cpb_dl_close(void* h) {
  auto* L = (Loader*)h;
  if (L) { L->close_shard(); delete L; }
}
