// strixw: the converted-weights file the serving path loads (formats/strixw.hpp:17-50) - reader, validation, and the
// device-resident copy with the quantized views the MoE kernels take (runtime/strixw_loader.hpp:37-75).
//
// Layout (formats/strixw.cpp:258-340): a 128-byte header {magic "STRIXWT\0", u32 version, u32 header bytes, u64 index offset,
// u64 index bytes, u64 data offset, u64 file bytes, u64 index hash, ..., u64 header hash at byte 120}, the index (metadata
// pairs, then one record per tensor: name, encoding, shape, group size, expert count, source parts, components {role, offset,
// bytes, hash}), then the data, every tensor 4096-aligned and every component 256-aligned, each already in its kernel's
// layout: Q4 / Q8 row-major = {q, scale, min} exactly as SxbQView wants them.
//
// Expert stacks (formats/merge_plan.cpp:33-41): "<layer>mlp.experts_gate_up" and "<layer>mlp.experts_down" hold the E routed
// experts and - when the shared expert has the same format - the shared expert as expert #E; "<layer>mlp.router" holds the
// E router rows and the shared gate's row, [E + 1, d].  sxb_strixw_expert_views cuts such a stack into the routed view and
// the shared expert's view without moving a byte.
//
// Loading (sxb_strixw_load): the file's whole data region becomes ONE device allocation (made here, once, at load time);
// components keep their file offsets, so their alignment carries over.  The bytes go through two pinned staging buffers
// filled by pread() and drained by asynchronous copies, a buffer being refilled only after the event behind its previous
// copy has completed.

#include "common.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace sxb {
namespace {

constexpr char kMagic[8] = {'S', 'T', 'R', 'I', 'X', 'W', 'T', '\0'};
constexpr uint32_t kVersion = 4, kOldestVersion = 1;
constexpr uint64_t kHeaderBytes = 128, kTensorAlign = 4096, kComponentAlign = 256;
constexpr uint64_t kK1 = 0x9e3779b97f4a7c15ull, kK2 = 0xd6e8feb86659fd93ull;

// formats/strixw.cpp:36-39, 193-244: four multiply-xorshift lanes over 32-byte blocks, seeded by the length.
inline uint64_t mix(uint64_t h, uint64_t w) {
    h ^= w * kK1;
    return (h ^ (h >> 31)) * kK2;
}
uint64_t hash64(const void *data, size_t n) {
    const auto *p = static_cast<const uint8_t *>(data);
    uint64_t h[4] = {n ^ kK1, n ^ kK2, ~(uint64_t)n ^ kK1, ~(uint64_t)n ^ kK2};
    size_t left = n;
    for (; left >= 32; left -= 32, p += 32) {
        uint64_t w[4];
        std::memcpy(w, p, 32);
        for (int l = 0; l < 4; ++l) h[l] = mix(h[l], w[l]);
    }
    size_t i = 0;
    for (int lane = 0; i + 8 <= left; i += 8, ++lane) {
        uint64_t w;
        std::memcpy(&w, p + i, 8);
        h[lane] = mix(h[lane], w);
    }
    if (i < left) {
        uint64_t w = 0;
        std::memcpy(&w, p + i, left - i);
        h[0] = mix(h[0], w ^ ((uint64_t)(left - i) << 56));
    }
    uint64_t r = mix(mix(mix(h[0], h[1]), h[2]), h[3]);
    r ^= r >> 33;
    r *= kK1;
    return r ^ (r >> 29);
}

struct Component {
    int role;
    uint64_t offset, bytes, hash;
};
struct Part {
    std::string source;
    int64_t row_offset, rows;
};
struct Tensor {
    std::string name;
    int encoding = 0;
    std::vector<int64_t> shape;
    int64_t group_size = 0, experts = 0;
    std::vector<Part> parts;
    std::vector<Component> components;
};

enum { kEncQ4 = 1, kEncQ4Chunk = 2, kEncBF16 = 3, kEncF32 = 4, kEncI64 = 5, kEncQ8 = 6, kEncQ8Chunk = 7, kEncQ6 = 8, kEncQ5 = 9 };
enum { kRoleData = 0, kRoleQ = 1, kRoleScale = 2, kRoleMin = 3 };

const char *encoding_name(int e) {
    static const char *names[] = {"unknown", "q4", "q4-chunk-major", "bf16", "f32", "i64", "q8", "q8-chunk-major", "q6", "q5"};
    return e >= 1 && e <= 9 ? names[e] : names[0];
}
const char *role_name(int r) {
    static const char *names[] = {"data", "q", "scale", "min"};
    return r >= 0 && r <= 3 ? names[r] : "unknown";
}

// The components an encoding has for a shape, with their exact sizes (formats/strixw.cpp:127-190).  Empty = bad record.
std::vector<Component> expected_components(const Tensor &t, std::string *why) {
    int64_t n = 1;
    for (int64_t d : t.shape) {
        if (d < 1 || n > INT64_MAX / d) {
            *why = "bad shape";
            return {};
        }
        n *= d;
    }
    auto quantized = [&](int64_t q_bytes_per_row_num, int64_t q_bytes_per_row_den, int64_t k_multiple) -> std::vector<Component> {
        if (t.shape.size() != 2) {
            *why = "needs shape [N, K]";
            return {};
        }
        const int64_t N = t.shape[0], K = t.shape[1], G = t.group_size;
        if (!(G == 32 || G == 64 || G == 128) || K % G != 0 || K % k_multiple != 0) {
            *why = cat("K = ", K, " with group size ", G);
            return {};
        }
        return {{kRoleQ, 0, (uint64_t)(N * K * q_bytes_per_row_num / q_bytes_per_row_den), 0},
                {kRoleScale, 0, (uint64_t)(N * (K / G) * 2), 0},
                {kRoleMin, 0, (uint64_t)(N * (K / G) * 2), 0}};
    };
    switch (t.encoding) {
        case kEncQ4:
        case kEncQ4Chunk: return quantized(1, 2, 1);
        case kEncQ8:
        case kEncQ8Chunk: return quantized(1, 1, 1);
        case kEncQ6: return quantized(3, 4, 64);
        case kEncQ5: return quantized(5, 8, 128);
        case kEncBF16:
        case kEncF32:
        case kEncI64: {
            if (t.group_size != 0) {
                *why = "group size on an unquantized tensor";
                return {};
            }
            const int64_t es = t.encoding == kEncBF16 ? 2 : t.encoding == kEncF32 ? 4 : 8;
            return {{kRoleData, 0, (uint64_t)(n * es), 0}};
        }
    }
    *why = cat("unknown encoding ", t.encoding);
    return {};
}

struct Cursor {
    const uint8_t *p;
    size_t n, at = 0;
    bool ok = true;
    template <typename T> T get() {
        T v{};
        if (n - at < sizeof(T)) {
            ok = false;
            return v;
        }
        std::memcpy(&v, p + at, sizeof(T));
        at += sizeof(T);
        return v;
    }
    std::string str(size_t len) {
        if (n - at < len) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char *>(p + at), len);
        at += len;
        return s;
    }
};

}  // namespace
}  // namespace sxb

struct SxbStrixw {
    std::string path;
    int fd = -1;
    void *map = nullptr;
    uint64_t file_bytes = 0, data_offset = 0;
    std::map<std::string, std::string> meta;
    std::vector<sxb::Tensor> tensors;
    std::map<std::string, size_t> by_name;
    uint8_t *device = nullptr;  // the data region [data_offset, file_bytes) on the device, after sxb_strixw_load
    double load_seconds = 0;
};

using namespace sxb;

namespace sxb {
namespace {

int parse(SxbStrixw *f) {
    const std::string where = "strixw '" + f->path + "'";
    const auto *b = static_cast<const uint8_t *>(f->map);
    const uint64_t size = f->file_bytes;
    auto rd32 = [&](size_t off) { uint32_t v; std::memcpy(&v, b + off, 4); return v; };
    auto rd64 = [&](size_t off) { uint64_t v; std::memcpy(&v, b + off, 8); return v; };
    SXB_CHECK(std::memcmp(b, kMagic, 8) == 0, where, ": not a strixw file (bad magic)");
    const uint32_t version = rd32(8), hsize = rd32(12);
    SXB_CHECK(version >= kOldestVersion && version <= kVersion, where, ": format version ", version, ", this build reads ",
              kOldestVersion, "..", kVersion);
    SXB_CHECK(hsize == kHeaderBytes, where, ": header size ", hsize, ", expected ", kHeaderBytes);
    SXB_CHECK(rd64(120) == hash64(b, 120), where, ": header hash mismatch (corrupt header)");
    const uint64_t index_off = rd64(16), index_bytes = rd64(24), file_bytes = rd64(40);
    f->data_offset = rd64(32);
    SXB_CHECK(file_bytes == size, where, ": header says ", file_bytes, " bytes, the file has ", size, " (truncated or appended to)");
    SXB_CHECK(index_off == kHeaderBytes && index_bytes <= size - index_off, where, ": index at ", index_off, " (", index_bytes,
              " bytes) doesn't fit the ", size, "-byte file");
    SXB_CHECK(f->data_offset % kTensorAlign == 0 && f->data_offset >= index_off + index_bytes && f->data_offset <= size, where,
              ": data offset ", f->data_offset, " (index ends at ", index_off + index_bytes, ", alignment ", kTensorAlign, ")");
    SXB_CHECK(rd64(48) == hash64(b + index_off, index_bytes), where, ": index hash mismatch (corrupt index)");

    Cursor c{b + index_off, (size_t)index_bytes};
    const uint32_t nmeta = c.get<uint32_t>();
    for (uint32_t i = 0; i < nmeta && c.ok; ++i) {
        std::string k = c.str(c.get<uint16_t>());
        std::string v = c.str(c.get<uint32_t>());
        SXB_CHECK(!c.ok || f->meta.emplace(k, std::move(v)).second, where, ": metadata key '", k, "' twice");
    }
    const uint32_t ntensors = c.get<uint32_t>();
    SXB_CHECK(c.ok && ntensors >= 1, where, ": the index ends inside its metadata, or holds no tensors");
    std::vector<std::pair<uint64_t, uint64_t>> spans;
    for (uint32_t i = 0; i < ntensors; ++i) {
        Tensor t;
        t.name = c.str(c.get<uint16_t>());
        t.encoding = c.get<uint8_t>();
        const uint8_t ndim = c.get<uint8_t>();
        for (uint8_t d = 0; d < ndim && c.ok; ++d) t.shape.push_back(c.get<int64_t>());
        t.group_size = c.get<int64_t>();
        t.experts = c.get<int64_t>();
        const uint16_t nparts = c.get<uint16_t>();
        for (uint16_t p = 0; p < nparts && c.ok; ++p) {
            Part part;
            part.source = c.str(c.get<uint16_t>());
            part.row_offset = c.get<int64_t>();
            part.rows = c.get<int64_t>();
            t.parts.push_back(std::move(part));
        }
        const uint8_t ncomp = c.get<uint8_t>();
        for (uint8_t k = 0; k < ncomp && c.ok; ++k) {
            Component comp;
            comp.role = c.get<uint8_t>();
            comp.offset = c.get<uint64_t>();
            comp.bytes = c.get<uint64_t>();
            comp.hash = c.get<uint64_t>();
            t.components.push_back(comp);
        }
        SXB_CHECK(c.ok, where, ": the index ends inside the record of tensor ", i, " ('", t.name, "')");
        // formats/strixw.cpp:78-97 validate_record
        SXB_CHECK(!t.name.empty(), where, ": tensor with an empty name");
        SXB_CHECK(!t.shape.empty() && t.shape.size() <= 8, where, ": tensor '", t.name, "' has ", t.shape.size(), " dims, expected 1..8");
        std::string why;
        const std::vector<Component> want = expected_components(t, &why);
        SXB_CHECK(!want.empty(), where, ": tensor '", t.name, "' (", encoding_name(t.encoding), "): ", why);
        SXB_CHECK(t.experts >= 0 && (t.experts == 0 || t.shape[0] % t.experts == 0), where, ": tensor '", t.name, "': ", t.shape[0],
                  " rows don't split into ", t.experts, " experts");
        int64_t next = 0;
        for (const Part &p : t.parts) {
            SXB_CHECK(!p.source.empty() && p.rows >= 1 && p.row_offset == next, where, ": tensor '", t.name, "' part '", p.source,
                      "' at row ", p.row_offset, " (", p.rows, " rows), expected to start at row ", next);
            next += p.rows;
        }
        SXB_CHECK(t.parts.empty() || next == t.shape[0], where, ": tensor '", t.name, "' parts cover ", next, " rows of ", t.shape[0]);
        SXB_CHECK(want.size() == t.components.size(), where, ": tensor '", t.name, "' (", encoding_name(t.encoding), ") has ",
                  t.components.size(), " components, expected ", want.size());
        for (size_t k = 0; k < want.size(); ++k) {
            const Component &g = t.components[k];
            SXB_CHECK(g.role == want[k].role && g.bytes == want[k].bytes, where, ": tensor '", t.name, "' component ", k, " is ",
                      role_name(g.role), " of ", g.bytes, " bytes, expected ", role_name(want[k].role), " of ", want[k].bytes);
            SXB_CHECK(g.offset >= f->data_offset && g.offset <= size && g.offset % kComponentAlign == 0 && g.bytes <= size - g.offset,
                      where, ": tensor '", t.name, "' ", role_name(g.role), " at ", g.offset, " (", g.bytes,
                      " bytes) is outside the data region [", f->data_offset, ", ", size, ") or not ", kComponentAlign, "-aligned");
            spans.emplace_back(g.offset, g.offset + g.bytes);
        }
        SXB_CHECK(f->by_name.emplace(t.name, f->tensors.size()).second, where, ": tensor '", t.name, "' twice");
        f->tensors.push_back(std::move(t));
    }
    SXB_CHECK(c.at == c.n, where, ": ", c.n - c.at, " unread bytes after the last index record");
    std::sort(spans.begin(), spans.end());
    for (size_t i = 1; i < spans.size(); ++i)
        SXB_CHECK(spans[i].first >= spans[i - 1].second, where, ": components overlap at byte ", spans[i].first);
    return SXB_OK;
}

const Tensor *find_tensor(const SxbStrixw *f, const char *name) {
    auto it = f->by_name.find(name ? name : "");
    return it == f->by_name.end() ? nullptr : &f->tensors[it->second];
}

void fill_info(const Tensor &t, SxbStrixwTensor *out) {
    std::memset(out, 0, sizeof(*out));
    out->name = t.name.c_str();
    out->encoding = t.encoding;
    out->ndim = (int)t.shape.size();
    for (size_t i = 0; i < t.shape.size(); ++i) out->shape[i] = t.shape[i];
    out->group_size = t.group_size, out->experts = t.experts;
    out->n_parts = (int)t.parts.size();
    out->n_components = (int)t.components.size();
    for (size_t i = 0; i < t.components.size() && i < 3; ++i) {
        out->component_role[i] = t.components[i].role;
        out->component_offset[i] = t.components[i].offset;
        out->component_bytes[i] = t.components[i].bytes;
        out->component_hash[i] = t.components[i].hash;
    }
}

const Component *component(const Tensor &t, int role) {
    for (const Component &c : t.components)
        if (c.role == role) return &c;
    return nullptr;
}

}  // namespace
}  // namespace sxb

extern "C" {

uint64_t sxb_strix_hash64(const void *data, size_t n) { return hash64(data, n); }

int sxb_strixw_open(const char *path, SxbStrixw **out) {
    SXB_CHECK(path != nullptr && out != nullptr, "strixw_open: null pointer");
    const std::string where = std::string("strixw '") + path + "'";
    const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
    SXB_CHECK(fd >= 0, where, ": open failed: ", std::strerror(errno));
    struct stat st {};
    if (::fstat(fd, &st) != 0) {
        const int err = errno;
        ::close(fd);
        SXB_CHECK(false, where, ": fstat failed: ", std::strerror(err));
    }
    const uint64_t size = (uint64_t)st.st_size;
    if (size < kHeaderBytes) {
        ::close(fd);
        SXB_CHECK(false, where, ": ", size, " bytes, smaller than the ", kHeaderBytes, "-byte header");
    }
    void *map = ::mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        const int err = errno;
        ::close(fd);
        SXB_CHECK(false, where, ": mmap of ", size, " bytes failed: ", std::strerror(err));
    }
    auto *f = new SxbStrixw;
    f->path = path, f->fd = fd, f->map = map, f->file_bytes = size;
    if (int rc = parse(f)) {
        ::munmap(map, size);
        ::close(fd);
        delete f;
        return rc;
    }
    *out = f;
    return SXB_OK;
}

int sxb_strixw_close(SxbStrixw *f) {
    if (f == nullptr) return SXB_OK;
    if (f->device) cudaFree(f->device);
    if (f->map) ::munmap(f->map, f->file_bytes);
    if (f->fd >= 0) ::close(f->fd);
    delete f;
    return SXB_OK;
}

int64_t sxb_strixw_tensor_count(const SxbStrixw *f) { return f ? (int64_t)f->tensors.size() : 0; }

int sxb_strixw_tensor(const SxbStrixw *f, int64_t index, SxbStrixwTensor *out) {
    SXB_CHECK(f != nullptr && out != nullptr, "strixw_tensor: null pointer");
    SXB_CHECK(index >= 0 && index < (int64_t)f->tensors.size(), "strixw '", f->path, "': tensor index ", index, " of ", f->tensors.size());
    fill_info(f->tensors[(size_t)index], out);
    return SXB_OK;
}

int sxb_strixw_find(const SxbStrixw *f, const char *name, SxbStrixwTensor *out) {
    SXB_CHECK(f != nullptr && name != nullptr && out != nullptr, "strixw_find: null pointer");
    const Tensor *t = find_tensor(f, name);
    SXB_CHECK(t != nullptr, "strixw '", f->path, "': no tensor '", name, "' (", f->tensors.size(), " tensors)");
    fill_info(*t, out);
    return SXB_OK;
}

int sxb_strixw_part(const SxbStrixw *f, const char *name, int index, const char **source, int64_t *row_offset, int64_t *rows) {
    SXB_CHECK(f != nullptr && name != nullptr && source != nullptr && row_offset != nullptr && rows != nullptr, "strixw_part: null pointer");
    const Tensor *t = find_tensor(f, name);
    SXB_CHECK(t != nullptr, "strixw '", f->path, "': no tensor '", name, "'");
    SXB_CHECK(index >= 0 && index < (int)t->parts.size(), "strixw '", f->path, "': tensor '", name, "' has ", t->parts.size(), " parts, asked for ", index);
    *source = t->parts[(size_t)index].source.c_str(), *row_offset = t->parts[(size_t)index].row_offset, *rows = t->parts[(size_t)index].rows;
    return SXB_OK;
}

const char *sxb_strixw_meta(const SxbStrixw *f, const char *key) {
    if (f == nullptr || key == nullptr) return nullptr;
    auto it = f->meta.find(key);
    return it == f->meta.end() ? nullptr : it->second.c_str();
}

const void *sxb_strixw_data(const SxbStrixw *f, const char *name, int role) {
    if (f == nullptr) return nullptr;
    const Tensor *t = find_tensor(f, name);
    const Component *c = t ? component(*t, role) : nullptr;
    return c ? static_cast<const uint8_t *>(f->map) + c->offset : nullptr;
}

int sxb_strixw_verify(const SxbStrixw *f, int threads) {
    SXB_CHECK(f != nullptr, "strixw_verify: null file");
    SXB_CHECK(threads >= 1 && threads <= 1024, "strixw_verify: threads = ", threads);
    std::vector<std::pair<const Tensor *, const Component *>> work;
    for (const Tensor &t : f->tensors)
        for (const Component &c : t.components) work.emplace_back(&t, &c);
    std::atomic<size_t> next{0};
    std::mutex mu;
    std::string first;
    auto worker = [&] {
        for (size_t i; (i = next.fetch_add(1)) < work.size();) {
            const auto [t, c] = work[i];
            if (hash64(static_cast<const uint8_t *>(f->map) + c->offset, c->bytes) != c->hash) {
                std::lock_guard<std::mutex> lock(mu);
                if (first.empty()) first = cat("tensor '", t->name, "' ", role_name(c->role), " (", c->bytes, " bytes at ", c->offset, ")");
            }
        }
    };
    std::vector<std::thread> pool;
    for (int i = 0; i < threads; ++i) pool.emplace_back(worker);
    for (std::thread &th : pool) th.join();
    SXB_CHECK(first.empty(), "strixw '", f->path, "': hash mismatch in ", first, " - the file is corrupt");
    return SXB_OK;
}

}  // extern "C"

// ---- the device-resident copy (runtime/strixw_loader.hpp:37-60) ---------------------------------------------------

namespace sxb {
namespace {

constexpr size_t kStageBytes = 32u << 20;  // one pinned staging buffer

// pread of [offset, offset + bytes) of the file into dst, by `threads` readers on disjoint slices.
int read_range(const SxbStrixw *f, uint8_t *dst, uint64_t offset, size_t bytes, int threads) {
    std::atomic<int> failed{0};
    auto reader = [&](size_t lo, size_t hi) {
        while (lo < hi && !failed.load()) {
            const ssize_t r = ::pread(f->fd, dst + lo, hi - lo, (off_t)(offset + lo));
            if (r < 0 && errno == EINTR) continue;
            if (r <= 0) {
                failed = errno ? errno : EIO;
                return;
            }
            lo += (size_t)r;
        }
    };
    threads = (int)std::max<size_t>(1, std::min<size_t>((size_t)threads, bytes / (1u << 20) + 1));
    std::vector<std::thread> pool;
    const size_t per = (bytes + (size_t)threads - 1) / (size_t)threads;
    for (int t = 0; t < threads; ++t) {
        const size_t lo = std::min(bytes, per * (size_t)t), hi = std::min(bytes, lo + per);
        if (lo < hi) pool.emplace_back(reader, lo, hi);
    }
    for (std::thread &th : pool) th.join();
    SXB_CHECK(failed.load() == 0, "strixw '", f->path, "': pread at offset ", offset, " failed: ", std::strerror(failed.load()));
    return SXB_OK;
}

int view_of(const SxbStrixw *f, const Tensor &t, int64_t row0, int64_t rows, SxbQView *v) {
    const Component *q = component(t, kRoleQ), *s = component(t, kRoleScale), *m = component(t, kRoleMin);
    SXB_CHECK(q && s && m, "strixw '", f->path, "': tensor '", t.name, "' (", encoding_name(t.encoding), ") is not a quantized row-major weight");
    const int64_t K = t.shape[1], G = t.group_size;
    const int64_t qrow = t.encoding == kEncQ4 ? K / 2 : K;
    const uint8_t *base = f->device - f->data_offset;  // a component's device address = base + its file offset
    v->q = base + q->offset + row0 * qrow;
    v->scale = reinterpret_cast<const uint16_t *>(base + s->offset) + row0 * (K / G);
    v->minv = reinterpret_cast<const uint16_t *>(base + m->offset) + row0 * (K / G);
    v->N = rows, v->K = K, v->G = G;
    return SXB_OK;
}

}  // namespace
}  // namespace sxb

extern "C" {

int sxb_strixw_load(SxbStrixw *f, int read_threads, sxb_stream_t stream) {
    const char *fn = "strixw_load";
    SXB_CHECK(f != nullptr, fn, ": null file");
    SXB_CHECK(read_threads >= 1 && read_threads <= 256, fn, ": read_threads = ", read_threads);
    if (f->device != nullptr) return SXB_OK;
    const uint64_t bytes = f->file_bytes - f->data_offset;
    SXB_CHECK(bytes > 0, fn, ": '", f->path, "' has an empty data region");
    auto st = static_cast<cudaStream_t>(stream);
    uint8_t *dev = nullptr, *stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    SXB_CUDA(cudaMalloc(&dev, bytes), fn, ": ", bytes, " bytes of device memory for '", f->path, "'");
    int rc = SXB_OK;
    auto cleanup = [&](bool keep) {
        for (int i = 0; i < 2; ++i) {
            if (done[i]) cudaEventDestroy(done[i]);
            if (stage[i]) cudaFreeHost(stage[i]);
        }
        if (!keep) cudaFree(dev);
    };
    for (int i = 0; i < 2 && rc == SXB_OK; ++i) {
        if (cudaMallocHost(&stage[i], kStageBytes) != cudaSuccess || cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) != cudaSuccess)
            rc = fail_cuda(SXB_FILE_, __LINE__, __func__, cudaGetLastError(), "strixw_load: pinned staging buffers");
    }
    const auto t0 = std::chrono::steady_clock::now();
    int slot = 0;
    bool used[2] = {false, false};
    for (uint64_t at = 0; at < bytes && rc == SXB_OK; at += kStageBytes, slot ^= 1) {
        const size_t n = (size_t)std::min<uint64_t>(kStageBytes, bytes - at);
        // the staging buffer is refilled only after the copy that last read it has completed
        if (used[slot] && cudaEventSynchronize(done[slot]) != cudaSuccess)
            rc = fail_cuda(SXB_FILE_, __LINE__, __func__, cudaGetLastError(), "strixw_load: waiting for a staging buffer");
        if (rc == SXB_OK) rc = read_range(f, stage[slot], f->data_offset + at, n, read_threads);
        if (rc == SXB_OK && (cudaMemcpyAsync(dev + at, stage[slot], n, cudaMemcpyHostToDevice, st) != cudaSuccess ||
                             cudaEventRecord(done[slot], st) != cudaSuccess))
            rc = fail_cuda(SXB_FILE_, __LINE__, __func__, cudaGetLastError(), "strixw_load: copy to the device");
        used[slot] = true;
    }
    if (rc == SXB_OK && cudaStreamSynchronize(st) != cudaSuccess)
        rc = fail_cuda(SXB_FILE_, __LINE__, __func__, cudaGetLastError(), "strixw_load: finishing the copies");
    cleanup(rc == SXB_OK);
    if (rc != SXB_OK) return rc;
    f->device = dev;
    f->load_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return SXB_OK;
}

double sxb_strixw_load_seconds(const SxbStrixw *f) { return f ? f->load_seconds : 0.0; }

const void *sxb_strixw_device_ptr(const SxbStrixw *f, const char *name, int role) {
    if (f == nullptr || f->device == nullptr) return nullptr;
    const Tensor *t = find_tensor(f, name);
    const Component *c = t ? component(*t, role) : nullptr;
    return c ? f->device + (c->offset - f->data_offset) : nullptr;
}

int sxb_strixw_qview(const SxbStrixw *f, const char *name, int64_t N, int64_t K, SxbQView *view, int *bits) {
    const char *fn = "strixw_qview";
    SXB_CHECK(f != nullptr && name != nullptr && view != nullptr && bits != nullptr, fn, ": null pointer");
    SXB_CHECK(f->device != nullptr, fn, ": '", f->path, "' is not loaded onto the device (sxb_strixw_load)");
    const Tensor *t = find_tensor(f, name);
    SXB_CHECK(t != nullptr, "strixw '", f->path, "': no tensor '", name, "'");
    SXB_CHECK(t->encoding == kEncQ4 || t->encoding == kEncQ8, "strixw '", f->path, "': tensor '", name, "' is ", encoding_name(t->encoding),
              ", expected q4 or q8 row-major");
    SXB_CHECK(t->shape[0] == N && t->shape[1] == K, "strixw '", f->path, "': tensor '", name, "' is [", t->shape[0], ", ", t->shape[1],
              "], expected [", N, ", ", K, "]");
    *bits = t->encoding == kEncQ4 ? 4 : 8;
    return view_of(f, *t, 0, N, view);
}

int sxb_strixw_expert_views(const SxbStrixw *f, const char *name, int64_t E, SxbQView *routed, SxbQView *shared, int *bits) {
    const char *fn = "strixw_expert_views";
    SXB_CHECK(f != nullptr && name != nullptr && routed != nullptr && bits != nullptr, fn, ": null pointer");
    SXB_CHECK(f->device != nullptr, fn, ": '", f->path, "' is not loaded onto the device (sxb_strixw_load)");
    const Tensor *t = find_tensor(f, name);
    SXB_CHECK(t != nullptr, "strixw '", f->path, "': no tensor '", name, "'");
    SXB_CHECK(t->encoding == kEncQ4 || t->encoding == kEncQ8, "strixw '", f->path, "': tensor '", name, "' is ", encoding_name(t->encoding),
              ", expected q4 or q8 row-major");
    SXB_CHECK(t->experts == E || t->experts == E + 1, "strixw '", f->path, "': tensor '", name, "' stacks ", t->experts, " experts, expected ", E,
              " (or ", E + 1, " with the shared expert as the last)");
    const int64_t rows = t->shape[0] / t->experts;
    *bits = t->encoding == kEncQ4 ? 4 : 8;
    if (int rc = view_of(f, *t, 0, E * rows, routed)) return rc;
    if (shared != nullptr) {
        std::memset(shared, 0, sizeof(*shared));
        if (t->experts == E + 1)
            if (int rc = view_of(f, *t, E * rows, rows, shared)) return rc;
    }
    return SXB_OK;
}

}  // extern "C"
