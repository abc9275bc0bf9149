// Device probe: prints one JSON line {"devices": [...]} describing the CUDA devices visible to this process.
//
// The driver API (libcuda.so.1) and NVML (libnvidia-ml.so.1) are opened with dlopen, so the program starts and
// answers {"devices": []} on a machine without a GPU or a driver.  It creates no CUDA context: names, compute
// capability, memory size and PCI location come from cuDeviceGetAttribute / cuDeviceTotalMem, free memory from
// NVML (looked up by PCI bus id).  The serving process runs it as a child with a timeout, so a wedged driver
// costs a bounded wait instead of a hung server.
//
// Counterpart of the reference's native probe (discover/native_probe_linux.go: dlopen of the backend registry,
// the CUDA driver API and NVML in a child process that prints JSON).
//
// Build: g++ -O2 -std=c++17 -DB2_DEVQUERY_MAIN devquery.cpp -ldl -o devquery   (also compiled into the host library,
// where b2n_probe_json() is the entry point).
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>

namespace {

typedef int CUresult;
typedef int CUdevice;
typedef CUresult (*cuInit_t)(unsigned);
typedef CUresult (*cuDriverGetVersion_t)(int*);
typedef CUresult (*cuDeviceGetCount_t)(int*);
typedef CUresult (*cuDeviceGet_t)(CUdevice*, int);
typedef CUresult (*cuDeviceGetName_t)(char*, int, CUdevice);
typedef CUresult (*cuDeviceGetAttribute_t)(int*, int, CUdevice);
typedef CUresult (*cuDeviceTotalMem_t)(size_t*, CUdevice);
typedef struct { unsigned char bytes[16]; } CUuuid;
typedef CUresult (*cuDeviceGetUuid_t)(CUuuid*, CUdevice);

constexpr int ATTR_INTEGRATED = 18, ATTR_PCI_BUS = 33, ATTR_PCI_DEVICE = 34, ATTR_PCI_DOMAIN = 50, ATTR_CC_MAJOR = 75, ATTR_CC_MINOR = 76;

typedef void* nvmlDevice_t;
struct nvmlMemory_t { unsigned long long total, free, used; };
typedef int (*nvmlInit_t)();
typedef int (*nvmlShutdown_t)();
typedef int (*nvmlDeviceGetHandleByPciBusId_t)(const char*, nvmlDevice_t*);
typedef int (*nvmlDeviceGetMemoryInfo_t)(nvmlDevice_t, nvmlMemory_t*);

std::string json_escape(const char* s) {
    std::string o;
    for (; *s; s++) {
        const unsigned char c = (unsigned char)*s;
        if (c == '"' || c == '\\') { o += '\\'; o += (char)c; }
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += (char)c;
    }
    return o;
}

template <typename T>
T sym(void* lib, const char* name) { return lib ? (T)dlsym(lib, name) : nullptr; }

std::string probe() {
    std::string out = "{\"devices\": [";
    void* cuda = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!cuda) return out + "], \"error\": \"libcuda.so.1 not found\"}";
    auto init = sym<cuInit_t>(cuda, "cuInit");
    auto drv = sym<cuDriverGetVersion_t>(cuda, "cuDriverGetVersion");
    auto count = sym<cuDeviceGetCount_t>(cuda, "cuDeviceGetCount");
    auto get = sym<cuDeviceGet_t>(cuda, "cuDeviceGet");
    auto name = sym<cuDeviceGetName_t>(cuda, "cuDeviceGetName");
    auto attr = sym<cuDeviceGetAttribute_t>(cuda, "cuDeviceGetAttribute");
    auto total = sym<cuDeviceTotalMem_t>(cuda, "cuDeviceTotalMem_v2");
    auto uuid = sym<cuDeviceGetUuid_t>(cuda, "cuDeviceGetUuid");
    if (!init || !count || !get || !name || !attr || !total) return out + "], \"error\": \"driver API symbols missing\"}";
    const CUresult rc = init(0);
    if (rc != 0) {
        char b[64];
        snprintf(b, sizeof b, "], \"error\": \"cuInit failed with %d\"}", rc);
        return out + b;
    }
    int version = 0, n = 0;
    if (drv) drv(&version);
    if (count(&n) != 0) n = 0;

    void* nvml = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
    auto ninit = sym<nvmlInit_t>(nvml, "nvmlInit_v2");
    auto nshut = sym<nvmlShutdown_t>(nvml, "nvmlShutdown");
    auto nbybus = sym<nvmlDeviceGetHandleByPciBusId_t>(nvml, "nvmlDeviceGetHandleByPciBusId_v2");
    auto nmem = sym<nvmlDeviceGetMemoryInfo_t>(nvml, "nvmlDeviceGetMemoryInfo");
    const bool have_nvml = ninit && nbybus && nmem && ninit() == 0;

    for (int i = 0; i < n; i++) {
        CUdevice d;
        if (get(&d, i) != 0) continue;
        char nm[256] = {0};
        name(nm, sizeof nm - 1, d);
        int major = 0, minor = 0, integrated = 0, bus = 0, dev = 0, dom = 0;
        attr(&major, ATTR_CC_MAJOR, d);
        attr(&minor, ATTR_CC_MINOR, d);
        attr(&integrated, ATTR_INTEGRATED, d);
        attr(&bus, ATTR_PCI_BUS, d);
        attr(&dev, ATTR_PCI_DEVICE, d);
        attr(&dom, ATTR_PCI_DOMAIN, d);
        size_t tot = 0;
        total(&tot, d);
        unsigned long long free_b = tot;
        char pci[32];
        snprintf(pci, sizeof pci, "%08x:%02x:%02x.0", dom, bus, dev);
        if (have_nvml) {
            nvmlDevice_t h;
            nvmlMemory_t m;
            if (nbybus(pci, &h) == 0 && nmem(h, &m) == 0) free_b = m.free;
        }
        char id[64];
        CUuuid u;
        if (uuid && uuid(&u, d) == 0) {
            const unsigned char* b = u.bytes;
            snprintf(id, sizeof id, "GPU-%02x%02x%02x%02x-%02x%02x-%02x%02x-%02x%02x-%02x%02x%02x%02x%02x%02x", b[0], b[1], b[2], b[3], b[4], b[5],
                     b[6], b[7], b[8], b[9], b[10], b[11], b[12], b[13], b[14], b[15]);
        } else {
            snprintf(id, sizeof id, "GPU-%d", i);
        }
        char buf[1024];
        snprintf(buf, sizeof buf,
                 "%s{\"id\": \"%s\", \"index\": %d, \"library\": \"cuda\", \"name\": \"%s\", \"compute_major\": %d, \"compute_minor\": %d, "
                 "\"total_memory\": %llu, \"free_memory\": %llu, \"driver\": \"%d.%d\", \"pci_id\": \"%s\", \"integrated\": %s}",
                 i ? ", " : "", id, i, json_escape(nm).c_str(), major, minor, (unsigned long long)tot, free_b, version / 1000, (version % 1000) / 10,
                 pci, integrated ? "true" : "false");
        out += buf;
    }
    if (have_nvml && nshut) nshut();
    return out + "]}";
}

}  // namespace

// Writes the JSON (NUL-terminated, truncated to cap - 1 bytes) and returns its full length.
extern "C" __attribute__((visibility("default"))) int b2n_probe_json(char* buf, int cap) {
    const std::string s = probe();
    if (buf && cap > 0) {
        const int n = (int)s.size() < cap - 1 ? (int)s.size() : cap - 1;
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return (int)s.size();
}

#ifdef B2_DEVQUERY_MAIN
int main() {
    puts(probe().c_str());
    return 0;
}
#endif
