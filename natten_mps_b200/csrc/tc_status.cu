// Device-side status word of the tensor-core kernels and the host-side hooks around it.
//
// Every barrier wait in the tcgen05 kernels has a cycle budget.  A CTA whose wait runs out
// raises the status word of its device, drains (no further data is touched), frees its TMEM
// and exits; CTAs that start afterwards see the word and drain at once, so a kernel that gave
// up never leaves work half done silently: the word stays set until the host clears it.
#include "tc_kernels.cuh"

#include "tc_plan.cuh"

#include <atomic>

namespace natten {

__device__ int g_tc_status = 0;

namespace {
std::mutex g_status_mutex;
int* g_status_addr[64] = {nullptr};
std::atomic<long long> g_wait_budget{tc::kWaitBudgetCycles};
std::atomic<int> g_inject{0};
} // namespace

namespace tcplan {

int* status_ptr()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_addr[dev]) {
        int* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_tc_status) != cudaSuccess) return nullptr;
        g_status_addr[dev] = p;
    }
    return g_status_addr[dev];
}

long long debug_wait_budget() { return g_wait_budget.load(); }
int debug_inject() { return g_inject.load(); }

} // namespace tcplan

int tc_device_status()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

int tc_clear_status()
{
    const int zero = 0;
    return (int)cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
}

int tc_status_async(int* host_word, cudaStream_t s)
{
    int* p = tcplan::status_ptr();
    if (!p || !host_word) return (int)cudaErrorInvalidValue;
    return (int)cudaMemcpyAsync(host_word, p, sizeof(int), cudaMemcpyDeviceToHost, s);
}

void tc_debug_wait(long long budget_cycles, int inject)
{
    g_wait_budget.store(budget_cycles > 0 ? budget_cycles : tc::kWaitBudgetCycles);
    g_inject.store(inject);
}

} // namespace natten
