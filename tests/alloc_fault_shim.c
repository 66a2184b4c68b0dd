/*
 * Test-only LD_PRELOAD shim around cudaMalloc: counts the calls and, when told
 * to, makes the n-th next one fail with cudaErrorMemoryAllocation without
 * touching the device. Host-side fault injection in the manner of the
 * reference's tests/cuda_fail_alloc.c; nothing on the GPU faults. Built by
 * tests/test_alloc_faults_gpu.py with the C compiler, loaded only into the child
 * process that test starts.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stddef.h>

static long calls_seen;   /* cudaMalloc calls since the last reset */
static long fail_in = -1; /* >= 0: that many more calls succeed, then one fails */

void alloc_shim_reset(void)
{
    __atomic_store_n(&calls_seen, 0, __ATOMIC_SEQ_CST);
    __atomic_store_n(&fail_in, -1, __ATOMIC_SEQ_CST);
}

long alloc_shim_calls(void)
{
    return __atomic_load_n(&calls_seen, __ATOMIC_SEQ_CST);
}

/* after_successes = 0 fails the very next call */
void alloc_shim_fail_after(long after_successes)
{
    __atomic_store_n(&fail_in, after_successes, __ATOMIC_SEQ_CST);
}

int alloc_shim_pending(void)
{
    return __atomic_load_n(&fail_in, __ATOMIC_SEQ_CST) >= 0;
}

/* the runtime's signature, spelled without its headers */
int cudaMalloc(void **pointer, size_t bytes)
{
    static int (*real)(void **, size_t);
    __atomic_add_fetch(&calls_seen, 1, __ATOMIC_SEQ_CST);
    long left = __atomic_load_n(&fail_in, __ATOMIC_SEQ_CST);
    if (left >= 0) {
        __atomic_store_n(&fail_in, left - 1, __ATOMIC_SEQ_CST);
        if (left == 0) {
            *pointer = NULL;
            return 2; /* cudaErrorMemoryAllocation */
        }
    }
    if (!real)
        real = (int (*)(void **, size_t))dlsym(RTLD_NEXT, "cudaMalloc");
    return real ? real(pointer, bytes) : 999;
}
