// File-backed, memory-mapped command queue and key/value state store shared between a worker process
// and its agent.  They take the place of the two LMDB environments of the reference (bounded FIFO of
// msgpack commands: src/etha/tensor_bus/command_queue.py:23-396; state db with heartbeat / match /
// transfer-signal keys: src/etha/tensor_bus/agent.py:131-144,427-431,530-531,728-735), with the same
// observable behaviour: bounded capacity, FIFO order, contents survive close and reopen, many processes
// may open the same path, readers of the state store take no lock.
//
// Mutual exclusion between processes uses open-file-description locks (released by the kernel when a
// process dies, so a crashed peer cannot wedge the queue); threads sharing one handle use a mutex.
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <new>

namespace {

constexpr uint64_t kQueueMagic = 0x3151484d53414845ull;  // "EHASMHQ1"
constexpr uint64_t kKvMagic = 0x31564b4d53414845ull;     // "EHASMKV1"

struct FileLock {
  int fd;
  explicit FileLock(int fd_, bool exclusive = true) : fd(fd_) {
    struct flock fl;
    memset(&fl, 0, sizeof(fl));
    fl.l_type = exclusive ? F_WRLCK : F_RDLCK;
    fl.l_whence = SEEK_SET;
    while (fcntl(fd, F_OFD_SETLKW, &fl) != 0 && errno == EINTR) {}
  }
  ~FileLock() {
    struct flock fl;
    memset(&fl, 0, sizeof(fl));
    fl.l_type = F_UNLCK;
    fl.l_whence = SEEK_SET;
    fcntl(fd, F_OFD_SETLK, &fl);
  }
};

// ---------------------------------------------------------------------------------------------
// queue: [header][index ring: capacity x {offset,len}][data ring: data_bytes]
// ---------------------------------------------------------------------------------------------
struct QHeader {
  uint64_t magic;
  uint64_t capacity;
  uint64_t data_bytes;
  uint64_t head;       // logical position of the oldest message
  uint64_t tail;       // logical position one past the newest message
  uint64_t data_head;  // byte offset (mod data_bytes) of the oldest message's data
  uint64_t data_tail;  // byte offset where the next message's data goes
  uint64_t data_used;  // bytes held (including skipped wrap padding)
};
struct QSlot { uint64_t offset, len, pad; };

struct Queue {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t map_bytes = 0;
  std::mutex mu;
  QHeader* hdr() { return reinterpret_cast<QHeader*>(map); }
  QSlot* slots() { return reinterpret_cast<QSlot*>(map + sizeof(QHeader)); }
  uint8_t* data() { return map + sizeof(QHeader) + hdr()->capacity * sizeof(QSlot); }
};

// ---------------------------------------------------------------------------------------------
// kv: [header][nslots x slot]; linear probing, per-slot sequence counter for lock-free readers
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kKeyCap = 184, kValCap = 2048;
struct KvHeader { uint64_t magic, nslots, count, pad; };
struct KvSlot {
  std::atomic<uint32_t> seq;  // odd while a writer is inside
  uint32_t state;             // 0 empty, 1 used, 2 deleted
  uint32_t klen, vlen;
  char key[kKeyCap];
  char val[kValCap];
};
struct Kv {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t map_bytes = 0;
  bool writable = true;
  std::mutex mu;
  KvHeader* hdr() { return reinterpret_cast<KvHeader*>(map); }
  KvSlot* slots() { return reinterpret_cast<KvSlot*>(map + sizeof(KvHeader)); }
};

uint64_t fnv1a(const char* p, uint32_t n) {
  uint64_t h = 1469598103934665603ull;
  for (uint32_t i = 0; i < n; ++i) { h ^= (uint8_t)p[i]; h *= 1099511628211ull; }
  return h;
}

}  // namespace

extern "C" {

// ---- queue --------------------------------------------------------------------------------------
void* etha_q_open(const char* path, uint64_t capacity, uint64_t data_bytes, int* err) {
  int fd = open(path, O_RDWR | O_CREAT, 0600);
  if (fd < 0) { if (err) *err = errno; return nullptr; }
  Queue* q = new (std::nothrow) Queue();
  q->fd = fd;
  {
    FileLock lock(fd);
    struct stat st;
    fstat(fd, &st);
    QHeader existing;
    bool fresh = st.st_size < (off_t)sizeof(QHeader) || pread(fd, &existing, sizeof(existing), 0) != (ssize_t)sizeof(existing) ||
                 existing.magic != kQueueMagic;
    if (!fresh) { capacity = existing.capacity; data_bytes = existing.data_bytes; }
    size_t total = sizeof(QHeader) + capacity * sizeof(QSlot) + data_bytes;
    if (fresh && ftruncate(fd, (off_t)total) != 0) { if (err) *err = errno; close(fd); delete q; return nullptr; }
    void* m = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (m == MAP_FAILED) { if (err) *err = errno; close(fd); delete q; return nullptr; }
    q->map = (uint8_t*)m;
    q->map_bytes = total;
    if (fresh) {
      QHeader* h = q->hdr();
      memset(h, 0, sizeof(*h));
      h->capacity = capacity;
      h->data_bytes = data_bytes;
      h->magic = kQueueMagic;
    }
  }
  if (err) *err = 0;
  return q;
}

// Returns the logical position (>= 0), -1 if `capacity` messages are queued, -2 if the data ring is full,
// -3 if the message can never fit.
int64_t etha_q_push(void* h, const void* buf, uint64_t len) {
  Queue* q = (Queue*)h;
  std::lock_guard<std::mutex> g(q->mu);
  FileLock lock(q->fd);
  QHeader* H = q->hdr();
  if (len > H->data_bytes / 2) return -3;
  if (H->tail - H->head >= H->capacity) return -1;
  uint64_t off = H->data_tail, pad = 0;
  if (off + len > H->data_bytes) { pad = H->data_bytes - off; off = 0; }  // no message straddles the end
  if (H->data_used + pad + len > H->data_bytes) return -2;
  memcpy(q->data() + off, buf, len);
  QSlot& s = q->slots()[H->tail % H->capacity];
  s.offset = off;
  s.len = len;
  s.pad = pad;
  H->data_tail = (off + len) % H->data_bytes;
  H->data_used += pad + len;
  std::atomic_thread_fence(std::memory_order_release);
  return (int64_t)(H->tail++);
}

// pop (consume != 0) or peek the oldest message. 0 ok, 1 empty, -3 buffer too small (*len = needed).
int etha_q_front(void* h, void* out, uint64_t cap, uint64_t* len, int consume) {
  Queue* q = (Queue*)h;
  std::lock_guard<std::mutex> g(q->mu);
  FileLock lock(q->fd);
  QHeader* H = q->hdr();
  if (H->tail == H->head) return 1;
  QSlot& s = q->slots()[H->head % H->capacity];
  *len = s.len;
  if (s.len > cap) return -3;
  memcpy(out, q->data() + s.offset, s.len);
  if (consume) {
    H->data_used -= s.pad + s.len;
    H->data_head = (s.offset + s.len) % H->data_bytes;
    H->head++;
    if (H->head == H->tail) { H->data_head = H->data_tail = 0; H->data_used = 0; }
  }
  return 0;
}

int64_t etha_q_size(void* h) {
  Queue* q = (Queue*)h;
  std::lock_guard<std::mutex> g(q->mu);
  FileLock lock(q->fd, false);
  return (int64_t)(q->hdr()->tail - q->hdr()->head);
}

uint64_t etha_q_capacity(void* h) { return ((Queue*)h)->hdr()->capacity; }

int etha_q_clear(void* h) {
  Queue* q = (Queue*)h;
  std::lock_guard<std::mutex> g(q->mu);
  FileLock lock(q->fd);
  QHeader* H = q->hdr();
  H->head = H->tail = 0;
  H->data_head = H->data_tail = H->data_used = 0;
  return 0;
}

int etha_q_close(void* h) {
  Queue* q = (Queue*)h;
  if (!q) return 0;
  if (q->map) { msync(q->map, q->map_bytes, MS_ASYNC); munmap(q->map, q->map_bytes); }
  if (q->fd >= 0) close(q->fd);
  delete q;
  return 0;
}

// ---- key/value state store -----------------------------------------------------------------------
void* etha_kv_open(const char* path, int create, int readonly, uint64_t nslots, int* err) {
  int fd = open(path, (readonly ? O_RDONLY : O_RDWR) | (create ? O_CREAT : 0), 0600);
  if (fd < 0) { if (err) *err = errno; return nullptr; }
  Kv* kv = new (std::nothrow) Kv();
  kv->fd = fd;
  kv->writable = !readonly;
  struct stat st;
  KvHeader existing;
  bool fresh;
  {
    // a reader never takes the lock: it only maps a file whose header is complete
    fstat(fd, &st);
    fresh = st.st_size < (off_t)sizeof(KvHeader) || pread(fd, &existing, sizeof(existing), 0) != (ssize_t)sizeof(existing) ||
            existing.magic != kKvMagic;
  }
  if (fresh && (readonly || !create)) { if (err) *err = ENOENT; close(fd); delete kv; return nullptr; }
  if (!fresh) nslots = existing.nslots;
  size_t total = sizeof(KvHeader) + nslots * sizeof(KvSlot);
  if (fresh) {
    FileLock lock(fd);
    if (ftruncate(fd, (off_t)total) != 0) { if (err) *err = errno; close(fd); delete kv; return nullptr; }
  }
  void* m = mmap(nullptr, total, readonly ? PROT_READ : (PROT_READ | PROT_WRITE), MAP_SHARED, fd, 0);
  if (m == MAP_FAILED) { if (err) *err = errno; close(fd); delete kv; return nullptr; }
  kv->map = (uint8_t*)m;
  kv->map_bytes = total;
  if (fresh) {
    FileLock lock(fd);
    KvHeader* H = kv->hdr();
    H->nslots = nslots;
    H->count = 0;
    std::atomic_thread_fence(std::memory_order_release);
    H->magic = kKvMagic;
  }
  if (err) *err = 0;
  return kv;
}

static KvSlot* kv_find(Kv* kv, const char* key, uint32_t klen, bool for_insert) {
  KvHeader* H = kv->hdr();
  uint64_t i = fnv1a(key, klen) % H->nslots;
  KvSlot* first_free = nullptr;
  for (uint64_t n = 0; n < H->nslots; ++n, i = (i + 1) % H->nslots) {
    KvSlot* s = &kv->slots()[i];
    if (s->state == 0) return for_insert ? (first_free ? first_free : s) : nullptr;
    if (s->state == 2) { if (!first_free) first_free = s; continue; }
    if (s->klen == klen && memcmp(s->key, key, klen) == 0) return s;
  }
  return for_insert ? first_free : nullptr;
}

int etha_kv_put(void* h, const char* key, uint32_t klen, const char* val, uint32_t vlen) {
  Kv* kv = (Kv*)h;
  if (!kv->writable) return -EACCES;
  if (klen > kKeyCap || vlen > kValCap) return -E2BIG;
  std::lock_guard<std::mutex> g(kv->mu);
  FileLock lock(kv->fd);
  KvSlot* s = kv_find(kv, key, klen, true);
  if (!s) return -ENOSPC;
  s->seq.fetch_add(1, std::memory_order_acq_rel);  // odd: write in progress
  if (s->state != 1) { memcpy(s->key, key, klen); s->klen = klen; kv->hdr()->count++; }
  memcpy(s->val, val, vlen);
  s->vlen = vlen;
  s->state = 1;
  s->seq.fetch_add(1, std::memory_order_release);
  return 0;
}

// 0 found, 1 missing, -E2BIG if `cap` is too small. Lock-free: retries while a writer is inside the slot.
int etha_kv_get(void* h, const char* key, uint32_t klen, char* out, uint32_t cap, uint32_t* vlen) {
  Kv* kv = (Kv*)h;
  for (int attempt = 0; attempt < 1000000; ++attempt) {
    KvSlot* s = kv_find(kv, key, klen, false);
    if (!s) return 1;
    uint32_t a = s->seq.load(std::memory_order_acquire);
    if (a & 1) continue;
    uint32_t n = s->vlen;
    bool used = s->state == 1 && s->klen == klen && memcmp(s->key, key, klen) == 0;
    if (n > kValCap) continue;
    if (used && n <= cap) memcpy(out, s->val, n);
    std::atomic_thread_fence(std::memory_order_acquire);
    if (s->seq.load(std::memory_order_relaxed) != a) continue;
    if (!used) return 1;
    *vlen = n;
    return n <= cap ? 0 : -E2BIG;
  }
  return -EBUSY;
}

int etha_kv_del(void* h, const char* key, uint32_t klen) {
  Kv* kv = (Kv*)h;
  if (!kv->writable) return -EACCES;
  std::lock_guard<std::mutex> g(kv->mu);
  FileLock lock(kv->fd);
  KvSlot* s = kv_find(kv, key, klen, false);
  if (!s) return 1;
  s->seq.fetch_add(1, std::memory_order_acq_rel);
  s->state = 2;
  kv->hdr()->count--;
  s->seq.fetch_add(1, std::memory_order_release);
  return 0;
}

int64_t etha_kv_count(void* h) { return (int64_t)((Kv*)h)->hdr()->count; }

int etha_kv_close(void* h) {
  Kv* kv = (Kv*)h;
  if (!kv) return 0;
  if (kv->map) munmap(kv->map, kv->map_bytes);
  if (kv->fd >= 0) close(kv->fd);
  delete kv;
  return 0;
}

}  // extern "C"
