// memory::Device / SynchronizedMemory for the lazy front end
// (reference: dali/array/memory/{device,synchronized_memory,memory_ops}.*).
// Host memory is a staging place only; device memory comes from the C ABI's
// pool (dalib200_alloc) and every size is 64-bit.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../../include/dali_b200.h"
#include "dali/array/expression/expression.h"

namespace memory {

static const int kMaxGpus = 16;   // DALI_MAX_GPU_DEVICES in the reference's config.h

Device default_preferred_device = Device::gpu(0);

WithDevicePreference::WithDevicePreference(Device device) : old_value(default_preferred_device) {
    default_preferred_device = device;
}
WithDevicePreference::~WithDevicePreference() { default_preferred_device = old_value; }

int Device::num_gpus() {
    try {
        lazy::ensure_backend();
    } catch (const std::runtime_error&) {
        return 0;
    }
    return dalib200_device_count();
}

std::vector<Device> Device::installed_devices() {
    std::vector<Device> out;
    out.push_back(Device::cpu());
    int n = num_gpus();
    for (int i = 0; i < n; ++i) out.push_back(Device::gpu(i));
    return out;
}

std::ostream& operator<<(std::ostream& os, const Device& d) {
    if (d.is_cpu()) return os << "cpu";
    if (d.is_gpu()) return os << "gpu/" << d.number();
    return os << "device?";
}

struct SynchronizedMemory::Impl {
    void* host = nullptr;
    bool host_fresh = false;
    void* dev[kMaxGpus] = {nullptr};
    bool dev_fresh[kMaxGpus] = {false};
    bool host_borrowed = false;
    bool dev_borrowed[kMaxGpus] = {false};
    bool clear_pending = false;
    uint64_t version = 0;
    std::shared_ptr<void> derived;
    uint64_t derived_version = 0;
};

SynchronizedMemory::SynchronizedMemory(size_t total, int inner, Device preferred, bool clear_on_allocation)
    : total_memory(total), inner_dimension(inner), preferred_device(preferred), impl_(new Impl()) {
    impl_->clear_pending = clear_on_allocation;
}

SynchronizedMemory::~SynchronizedMemory() {
    if (impl_->host && !impl_->host_borrowed) std::free(impl_->host);
    for (int g = 0; g < kMaxGpus; ++g)
        if (impl_->dev[g] && !impl_->dev_borrowed[g]) dalib200_free(g, impl_->dev[g], total_memory);
    delete impl_;
}

bool SynchronizedMemory::is_fresh(const Device& d) const {
    if (d.is_cpu()) return impl_->host_fresh;
    if (d.is_gpu() && d.number() >= 0 && d.number() < kMaxGpus) return impl_->dev_fresh[d.number()];
    return false;
}
int SynchronizedMemory::fresh_gpu() const {
    for (int g = 0; g < kMaxGpus; ++g)
        if (impl_->dev_fresh[g]) return g;
    return -1;
}
bool SynchronizedMemory::is_allocated(const Device& d) const {
    if (d.is_cpu()) return impl_->host != nullptr;
    if (d.is_gpu() && d.number() >= 0 && d.number() < kMaxGpus) return impl_->dev[d.number()] != nullptr;
    return false;
}
bool SynchronizedMemory::is_any_fresh() const {
    if (impl_->host_fresh) return true;
    for (int g = 0; g < kMaxGpus; ++g) if (impl_->dev_fresh[g]) return true;
    return false;
}

uint64_t SynchronizedMemory::version() const { return impl_->version; }
std::shared_ptr<void>& SynchronizedMemory::derived_data() { return impl_->derived; }
uint64_t& SynchronizedMemory::derived_version() { return impl_->derived_version; }

void SynchronizedMemory::clear() {
    ++impl_->version;
    impl_->host_fresh = false;
    for (int g = 0; g < kMaxGpus; ++g) impl_->dev_fresh[g] = false;
    impl_->clear_pending = true;
}


void* SynchronizedMemory::data(const Device& device, AM mode) {
    DALI_ASSERT(device.is_cpu() || (device.is_gpu() && device.number() >= 0 && device.number() < kMaxGpus),
                "SynchronizedMemory::data: unknown device");
    Impl* m = impl_;
    const int g = device.number();
    // allocate
    void*& here = device.is_cpu() ? m->host : m->dev[g];
    if (!here) {
        if (device.is_cpu()) {
            here = std::malloc(total_memory ? total_memory : 1);
            DALI_ASSERT(here, "out of host memory");
        } else {
            lazy::ensure_backend();
            lazy::check(dalib200_alloc(g, total_memory, &here), "dalib200_alloc");
        }
    }
    bool& fresh_here = device.is_cpu() ? m->host_fresh : m->dev_fresh[g];
    if (!fresh_here) {
        if (!is_any_fresh()) {
            // first touch: zero if asked to, else leave uninitialised
            if (m->clear_pending) {
                if (device.is_cpu()) std::memset(here, 0, total_memory);
                else lazy::check(dalib200_memset(g, here, 0, total_memory, nullptr), "dalib200_memset");
                m->clear_pending = false;
            }
        } else if (mode != AM_OVERWRITE) {
            // bring a fresh copy here
            if (device.is_cpu()) {
                int src = -1;
                for (int k = 0; k < kMaxGpus; ++k) if (m->dev_fresh[k]) { src = k; break; }
                lazy::check(dalib200_memcpy_d2h(src, here, m->dev[src], total_memory, nullptr), "dalib200_memcpy_d2h");
                lazy::check(dalib200_sync(src, nullptr), "dalib200_sync");
            } else if (m->host_fresh) {
                lazy::check(dalib200_memcpy_h2d(g, here, m->host, total_memory, nullptr), "dalib200_memcpy_h2d");
                // A pageable host buffer has been staged by the time the call returns.  A page-locked one (borrow_host,
                // dalib200_host_alloc) is read asynchronously by the copy engine: its owner must leave it untouched until
                // a synchronising call has returned, and borrow it again after a host-side write (the device copy is
                // marked fresh here and is not refreshed behind the caller's back).
            } else {
                // fresh on another GPU only: stage through the host (the reference asserts here,
                // dali/array/memory/memory_ops.cu.cpp:120-125)
                data(Device::cpu(), AM_READONLY);
                lazy::check(dalib200_memcpy_h2d(g, here, m->host, total_memory, nullptr), "dalib200_memcpy_h2d");
            }
        }
        fresh_here = true;
    }
    if (mode != AM_READONLY) {
        ++m->version;
        m->host_fresh = false;
        for (int k = 0; k < kMaxGpus; ++k) m->dev_fresh[k] = false;
        fresh_here = true;
    }
    return here;
}

const void* SynchronizedMemory::readonly_data(const Device& d) { return data(d, AM_READONLY); }
void* SynchronizedMemory::mutable_data(const Device& d) { return data(d, AM_MUTABLE); }
void* SynchronizedMemory::overwrite_data(const Device& d) { return data(d, AM_OVERWRITE); }
void SynchronizedMemory::to_device(const Device& d) { data(d, AM_READONLY); }

void SynchronizedMemory::adopt_buffer(const Device& device, void* buffer) {
    Impl* m = impl_;
    DALI_ASSERT(!is_allocated(device), "adopt_buffer: this memory already owns a buffer on that device");
    ++m->version;
    if (device.is_cpu()) { m->host = buffer; m->host_fresh = true; }
    else { m->dev[device.number()] = buffer; m->dev_fresh[device.number()] = true; }
}

void SynchronizedMemory::borrow_buffer(const Device& device, void* buffer) {
    adopt_buffer(device, buffer);
    if (device.is_cpu()) impl_->host_borrowed = true;
    else impl_->dev_borrowed[device.number()] = true;
}

void SynchronizedMemory::disown_buffer(const Device& device) {
    Impl* m = impl_;
    if (device.is_cpu()) { m->host = nullptr; m->host_fresh = false; }
    else { m->dev[device.number()] = nullptr; m->dev_fresh[device.number()] = false; }
}

}  // namespace memory
