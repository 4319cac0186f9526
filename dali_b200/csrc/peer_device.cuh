// Device side of the peer exchange (see peer.h): system-scope flag stores and loads,
// a bounded wait.  No host headers: this text is also spliced in front of the device
// prelude of every run-time generated kernel.
#ifndef DALI_B200_CSRC_PEER_DEVICE_CUH
#define DALI_B200_CSRC_PEER_DEVICE_CUH

__device__ __forceinline__ unsigned long long dali_peer_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// flag = epoch, visible to every GPU after everything this thread (and, through the CTA
// barrier before it, this CTA) has written
__device__ __forceinline__ void dali_peer_flag_release(unsigned long long* flag, unsigned long long epoch) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(epoch) : "memory");
}

__device__ __forceinline__ unsigned long long dali_peer_flag_acquire(const unsigned long long* flag) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
    return v;
}

// Waits until *flag >= epoch.  Gives up after wait_ns (returns false and raises *error): a rank that never
// arrives must not hang this GPU.  The caller carries on with whatever its block holds and the host reads
// the error word (dalib200_comm_error_flag).
__device__ __forceinline__ bool dali_peer_wait(const unsigned long long* flag, unsigned long long epoch,
                                               unsigned long long wait_ns, int* error) {
    if (dali_peer_flag_acquire(flag) >= epoch) return true;
    const unsigned long long t0 = dali_peer_now_ns();
    unsigned spins = 0;
    while (dali_peer_flag_acquire(flag) < epoch) {
        if (++spins > 64) __nanosleep(spins > 4096 ? 2000 : 100);
        if ((spins & 63) == 0 && dali_peer_now_ns() - t0 > wait_ns) {
            if (dali_peer_flag_acquire(flag) >= epoch) return true;
            atomicExch(error, 1);
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ unsigned long long* dali_peer_flag(char* block, int parity, int rank, int chunk) {
    return reinterpret_cast<unsigned long long*>(block + DALI_PEER_OFF_FLAGS) +
           ((unsigned long long)(parity * DALI_PEER_MAX_WORLD + rank) * DALI_PEER_CHUNKS + chunk);
}
__device__ __forceinline__ char* dali_peer_slot(char* block, int parity, int rank) {
    return block + DALI_PEER_OFF_DATA + (unsigned long long)(parity * DALI_PEER_MAX_WORLD + rank) * DALI_PEER_SLOT_BYTES;
}
__device__ __forceinline__ unsigned long long* dali_peer_fused_flag(char* block, int parity, int rank) {
    return reinterpret_cast<unsigned long long*>(block + DALI_PEER_OFF_FUSED_FLAGS) + (parity * DALI_PEER_MAX_WORLD + rank);
}
__device__ __forceinline__ char* dali_peer_fused_slot(char* block, int parity, int rank) {
    return block + DALI_PEER_OFF_FUSED_DATA + (unsigned long long)(parity * DALI_PEER_MAX_WORLD + rank) * DALI_PEER_FUSED_SLOT_BYTES;
}

#endif
