// The per-handle device-memory arena (see nb_internal.h for why every buffer lives in one).
#include "nb_internal.h"

namespace nb {

namespace {
constexpr size_t ALIGN = 512;
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
thread_local std::shared_ptr<Arena> t_current;
}  // namespace

std::shared_ptr<Arena> &Arena::current() { return t_current; }

Arena::~Arena() {
    for (Chunk &c : chunks)
        if (c.base) (void)cudaFree(c.base);
}

void *Arena::alloc(size_t bytes) {
    const size_t len = round_up(std::max<size_t>(bytes, 1), ALIGN);
    for (int attempt = 0; attempt < 2; attempt++) {
        for (Chunk &c : chunks) {
            for (auto it = c.free.begin(); it != c.free.end(); ++it) {
                if (it->second < len) continue;
                const size_t off = it->first, rest = it->second - len;
                c.free.erase(it);
                if (rest) c.free[off + len] = rest;
                void *p = c.base + off;
                live[p] = {c.base, len};
                in_use += len;
                return p;
            }
        }
        if (attempt) break;
        // a new chunk: at least MIN_CHUNK, or the request plus the guards at both ends when that is larger
        const size_t need = round_up(len + 2 * END_GUARD, (size_t)2 << 20);
        size_t size = std::max(need, MIN_CHUNK);
        char *base = nullptr;
        cudaError_t e = cudaMalloc((void **)&base, size);
        if (e != cudaSuccess && size > need) {
            (void)cudaGetLastError();
            size = need;
            e = cudaMalloc((void **)&base, size);
        }
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            throw Error(NB_ERR_CUDA, std::string("cudaMalloc of a ") + std::to_string(size >> 20) + " MiB arena chunk: " +
                                         cudaGetErrorString(e));
        }
        Chunk c;
        c.base = base;
        c.size = size;
        c.free[END_GUARD] = size - 2 * END_GUARD;
        chunks.push_back(std::move(c));
    }
    throw Error(NB_ERR_CUDA, "arena: a fresh chunk could not hold the request");
}

void Arena::release(void *p) {
    auto lv = live.find(p);
    if (lv == live.end()) return;
    char *base = lv->second.first;
    size_t off = (char *)p - base, len = lv->second.second;
    live.erase(lv);
    in_use -= len;
    for (size_t ci = 0; ci < chunks.size(); ci++) {
        Chunk &c = chunks[ci];
        if (c.base != base) continue;
        auto next = c.free.lower_bound(off);
        if (next != c.free.end() && off + len == next->first) {         // merge with the run behind
            len += next->second;
            next = c.free.erase(next);
        }
        if (next != c.free.begin()) {                                   // ... and with the run in front
            auto prev = std::prev(next);
            if (prev->first + prev->second == off) {
                off = prev->first;
                len += prev->second;
                c.free.erase(prev);
            }
        }
        c.free[off] = len;
        // a chunk that is empty again goes back to the driver unless it is the only one
        if (chunks.size() > 1 && c.free.size() == 1 && c.free.begin()->second == c.size - 2 * END_GUARD) {
            (void)cudaFree(c.base);
            chunks.erase(chunks.begin() + ci);
        }
        return;
    }
}

}  // namespace nb
