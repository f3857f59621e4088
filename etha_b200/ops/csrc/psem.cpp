// POSIX named semaphores for Python (ctypes): create/open, post, timed wait, value, close, unlink.
// The reference reaches the same calls through the `posix_ipc` package (src/etha/tensor_bus/client.py:153-182,
// src/etha/tensor_bus/command_queue.py:38-80, src/etha/tensor_bus/agent.py:761-785).
#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <semaphore.h>
#include <time.h>

extern "C" {

// flags: bit0 = O_CREAT, bit1 = O_EXCL.  Returns the handle or null with *err = errno.
void* etha_sem_open(const char* name, int flags, unsigned initial, int* err) {
  int oflag = 0;
  if (flags & 1) oflag |= O_CREAT;
  if (flags & 2) oflag |= O_EXCL;
  sem_t* s = (oflag & O_CREAT) ? sem_open(name, oflag, 0600, initial) : sem_open(name, 0);
  if (s == SEM_FAILED) {
    if (err) *err = errno;
    return nullptr;
  }
  if (err) *err = 0;
  return s;
}

int etha_sem_post(void* h) { return sem_post((sem_t*)h) == 0 ? 0 : -errno; }

// timeout_s < 0: wait forever; == 0: try once. Returns 0 acquired, 1 timed out / would block, <0 -errno.
int etha_sem_wait(void* h, double timeout_s) {
  sem_t* s = (sem_t*)h;
  int rc;
  if (timeout_s < 0) {
    do { rc = sem_wait(s); } while (rc != 0 && errno == EINTR);
  } else if (timeout_s == 0) {
    rc = sem_trywait(s);
    if (rc != 0 && errno == EAGAIN) return 1;
  } else {
    timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    double whole = floor(timeout_s);
    ts.tv_sec += (time_t)whole;
    ts.tv_nsec += (long)((timeout_s - whole) * 1e9);
    if (ts.tv_nsec >= 1000000000L) { ts.tv_sec += 1; ts.tv_nsec -= 1000000000L; }
    do { rc = sem_timedwait(s, &ts); } while (rc != 0 && errno == EINTR);
    if (rc != 0 && errno == ETIMEDOUT) return 1;
  }
  return rc == 0 ? 0 : -errno;
}

int etha_sem_value(void* h, int* out) { return sem_getvalue((sem_t*)h, out) == 0 ? 0 : -errno; }
int etha_sem_close(void* h) { return sem_close((sem_t*)h) == 0 ? 0 : -errno; }
int etha_sem_unlink(const char* name) { return sem_unlink(name) == 0 ? 0 : -errno; }

}  // extern "C"
