/* windows.h — a minimal stand-in so that the reference's src/backends/cuda/moe_cpu_expert.c
 * (whose thread pool is written against Win32) compiles unmodified with gcc on Linux.
 * TEST INFRASTRUCTURE ONLY: used by oracle/Makefile to build oracle/_ref; never by the product.
 * Provides exactly the names that file uses: integer/handle typedefs, __declspec(align(n)),
 * __forceinline, SRWLOCK, Interlocked*, WaitOnAddress/WakeByAddressAll, CreateThread,
 * SetThreadPriority; and for tools/moe_cpu_bench/moe_cpu_bench.cu (oracle/ref_gpu_kernels.cu):
 * GetCurrentThread, SetThreadAffinityMask. */
#ifndef SP_ORACLE_WIN32_SHIM_H
#define SP_ORACLE_WIN32_SHIM_H
#include <stdint.h>
#include <stdlib.h>
#include <sched.h>
#include <pthread.h>
#include <cpuid.h>
#include <immintrin.h>

typedef long LONG;
typedef unsigned long DWORD;
typedef void *HANDLE;
typedef void *LPVOID;
typedef void *PVOID;
#define WINAPI
#define INFINITE 0xFFFFFFFFu
#define THREAD_PRIORITY_ABOVE_NORMAL 1
#define __declspec(x) __attribute__((x))
#define align(n) aligned(n)
#define __forceinline inline __attribute__((always_inline))

typedef struct { pthread_mutex_t m; } SRWLOCK;
#define SRWLOCK_INIT { PTHREAD_MUTEX_INITIALIZER }
static inline void AcquireSRWLockExclusive(SRWLOCK *l) { pthread_mutex_lock(&l->m); }
static inline void ReleaseSRWLockExclusive(SRWLOCK *l) { pthread_mutex_unlock(&l->m); }

static inline LONG InterlockedIncrement(volatile LONG *p) { return __atomic_add_fetch(p, 1, __ATOMIC_SEQ_CST); }
static inline LONG InterlockedExchange(volatile LONG *p, LONG v) { return __atomic_exchange_n(p, v, __ATOMIC_SEQ_CST); }
/* parked workers simply yield and re-check: correct, if not as quiet as a futex */
static inline int WaitOnAddress(volatile void *a, void *cmp, size_t n, DWORD ms) { (void)a; (void)cmp; (void)n; (void)ms; sched_yield(); return 1; }
static inline void WakeByAddressAll(void *a) { (void)a; }

typedef DWORD (*LPTHREAD_START_ROUTINE)(LPVOID);
struct sp_shim_thr_arg { LPTHREAD_START_ROUTINE f; LPVOID a; };
static void *sp_shim_thr_tramp(void *p) { struct sp_shim_thr_arg t = *(struct sp_shim_thr_arg *)p; free(p); t.f(t.a); return 0; }
static inline HANDLE CreateThread(void *sa, size_t ss, LPTHREAD_START_ROUTINE f, LPVOID a, DWORD fl, DWORD *id) {
    (void)sa; (void)ss; (void)fl; (void)id;
    pthread_t *t = (pthread_t *)malloc(sizeof *t);
    struct sp_shim_thr_arg *ar = (struct sp_shim_thr_arg *)malloc(sizeof *ar);
    if (!t || !ar) { free(t); free(ar); return 0; }
    ar->f = f; ar->a = a;
    if (pthread_create(t, 0, sp_shim_thr_tramp, ar)) { free(t); free(ar); return 0; }
    pthread_detach(*t);
    return t;
}
static inline int SetThreadPriority(HANDLE h, int p) { (void)h; (void)p; return 1; }
static inline HANDLE GetCurrentThread(void) { return 0; }
static inline unsigned long long SetThreadAffinityMask(HANDLE h, unsigned long long m) { (void)h; return m; }
#endif
