// Context, error reporting, codebook loading, compressor threshold derivation, timers.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include "cn_internal.h"

#include <atomic>
static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void cn_count_launch(void) { g_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" uint64_t cn_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

void cn_set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cn_cuda_fail(cudaError_t e, const char *what)
{
    cn_set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return CN_ERR_CUDA;
}

extern "C" const char *cn_last_error(void) { return g_err; }

extern "C" const char *cn_status_string(int s)
{
    switch (s) {
        case CN_OK: return "CN_OK";
        case CN_ERR_ARG: return "CN_ERR_ARG";
        case CN_ERR_SHAPE: return "CN_ERR_SHAPE";
        case CN_ERR_CUDA: return "CN_ERR_CUDA";
        case CN_ERR_NCCL: return "CN_ERR_NCCL";
        case CN_ERR_TIMEOUT: return "CN_ERR_TIMEOUT";
        case CN_ERR_UNSUPPORTED: return "CN_ERR_UNSUPPORTED";
        case CN_ERR_NOMEM: return "CN_ERR_NOMEM";
    }
    return "CN_ERR_?";
}

extern "C" int cn_version(void) { return 100; }
extern "C" int cn_compiled_arch(void) { return 100; }

// ------------------------------------------------------------------------------------------------
// Minimal HDF5 reader for the files the reference reads with libhdf5 (read_hdf5 of dataset "/Default",
// source/util.cu:100-131): version-0 superblock, root group with a symbol table (B-tree + local heap), version-1
// object headers, a simple dataspace of rank 1 or 2, an integer or IEEE float datatype of 4 or 8 bytes (little
// endian), contiguous or compact layout.  That covers what numpy / h5py write for dense arrays, including the
// reference's codebook (source/8bit_floats.hdf5) and its test fixtures.  Everything is bounds-checked; anything
// else is reported as unsupported.
// ------------------------------------------------------------------------------------------------
namespace {
// The file is mapped read-only, not read: a data set of several GB is converted straight from the page cache.
struct H5 {
    const unsigned char *b = nullptr;
    uint64_t size = 0;
    ~H5() { if (b) munmap((void *)b, size); }
    H5() = default;
    H5(const H5 &) = delete;
    H5 &operator=(const H5 &) = delete;
    bool ok(uint64_t off, uint64_t len) const { return off <= size && len <= size - off; }
    uint64_t u(uint64_t off, int n) const
    {
        uint64_t v = 0;
        for (int i = n - 1; i >= 0; --i) v = (v << 8) | b[off + i];
        return v;
    }
};

struct H5Dataset {
    int rank = 0;
    uint64_t dims[2] = {1, 1};
    int type_class = -1, type_size = 0, type_signed = 0;
    uint64_t data_addr = 0, data_size = 0;
    bool have_space = false, have_type = false, have_layout = false;
};

bool h5_parse_messages(const H5 &f, uint64_t p, uint64_t end, int &left, H5Dataset &d, int depth)
{
    while (left > 0 && p + 8 <= end) {
        if (!f.ok(p, 8)) return false;
        const unsigned type = (unsigned)f.u(p, 2);
        const uint64_t size = f.u(p + 2, 2), body = p + 8;
        if (!f.ok(body, size)) return false;
        --left;
        if (type == 0x1 && size >= 8) {   // dataspace
            const int ver = f.b[body], rank = f.b[body + 1];
            const uint64_t dp = body + (ver == 1 ? 8 : 4);
            if (rank < 1 || rank > 2 || !f.ok(dp, 8ull * rank)) return false;
            d.rank = rank;
            for (int i = 0; i < rank; ++i) d.dims[i] = f.u(dp + 8ull * i, 8);
            d.have_space = true;
        } else if (type == 0x3 && size >= 8) {   // datatype
            d.type_class = f.b[body] & 0x0f;
            const unsigned bits0 = f.b[body + 1];
            if (bits0 & 1) return false;   // big endian
            d.type_signed = (bits0 >> 3) & 1;
            d.type_size = (int)f.u(body + 4, 4);
            d.have_type = true;
        } else if (type == 0x8 && size >= 2) {   // data layout
            const int ver = f.b[body], cls = f.b[body + 1];
            if (ver != 3) return false;
            if (cls == 1 && size >= 18) { d.data_addr = f.u(body + 2, 8); d.data_size = f.u(body + 10, 8); }
            else if (cls == 0 && size >= 4) { d.data_size = f.u(body + 2, 2); d.data_addr = body + 4; }
            else return false;   // chunked
            d.have_layout = true;
        } else if (type == 0x10 && size >= 16 && depth < 8) {   // header continuation
            const uint64_t off = f.u(body, 8), len = f.u(body + 8, 8);
            if (!f.ok(off, len) || !h5_parse_messages(f, off, off + len, left, d, depth + 1)) return false;
        }
        p = body + size;
    }
    return true;
}

// object-header address of `name` in the group whose B-tree / heap are given; 0 when not found
uint64_t h5_find(const H5 &f, uint64_t tree, uint64_t heap_data, const char *name, int depth)
{
    if (depth > 8 || !f.ok(tree, 24) || memcmp(&f.b[tree], "TREE", 4) != 0 || f.b[tree + 4] != 0) return 0;
    const int level = f.b[tree + 5], entries = (int)f.u(tree + 6, 2);
    for (int e = 0; e < entries; ++e) {
        const uint64_t cp = tree + 24 + 8 + 16ull * e;   // key0, child0, key1, child1, ...
        if (!f.ok(cp, 8)) return 0;
        const uint64_t child = f.u(cp, 8);
        if (level > 0) {
            const uint64_t r = h5_find(f, child, heap_data, name, depth + 1);
            if (r) return r;
            continue;
        }
        if (!f.ok(child, 8) || memcmp(&f.b[child], "SNOD", 4) != 0) return 0;
        const int nsym = (int)f.u(child + 6, 2);
        for (int k = 0; k < nsym; ++k) {
            const uint64_t ent = child + 8 + 40ull * k;
            if (!f.ok(ent, 40)) return 0;
            const uint64_t noff = heap_data + f.u(ent, 8);
            const size_t nl = strlen(name);
            if (f.ok(noff, nl + 1) && memcmp(&f.b[noff], name, nl + 1) == 0) return f.u(ent + 8, 8);
        }
    }
    return 0;
}
}  // namespace

namespace {
// Loads the file, finds the dataset and checks that its data lie inside the file; n = number of elements.
int h5_locate(const char *path, const char *dataset, H5 &f, H5Dataset &d, uint64_t &n)
{
    {
        const int fd = open(path, O_RDONLY);
        CN_REQUIRE(fd >= 0, CN_ERR_ARG, "cn_hdf5_read: cannot open %s", path);
        struct stat sb;
        const bool stat_ok = fstat(fd, &sb) == 0 && sb.st_size >= 96;
        void *m = stat_ok ? mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0) : MAP_FAILED;
        close(fd);
        CN_REQUIRE(stat_ok, CN_ERR_ARG, "cn_hdf5_read: %s is too short", path);
        CN_REQUIRE(m != MAP_FAILED, CN_ERR_ARG, "cn_hdf5_read: cannot map %s", path);
        f.b = (const unsigned char *)m;
        f.size = (uint64_t)sb.st_size;
    }
    static const unsigned char sig[8] = {0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};
    CN_REQUIRE(memcmp(f.b, sig, 8) == 0, CN_ERR_ARG, "cn_hdf5_read: %s has no HDF5 signature", path);
    CN_REQUIRE(f.b[8] == 0 && f.b[13] == 8 && f.b[14] == 8, CN_ERR_UNSUPPORTED,
               "cn_hdf5_read: %s: only version-0 superblocks with 8-byte offsets are read", path);
    // root symbol-table entry at byte 56: object header address, cache type, scratch = B-tree and heap addresses
    uint64_t tree = 0, heap = 0;
    if (f.u(72, 4) == 1) {
        tree = f.u(80, 8);
        heap = f.u(88, 8);
    } else {
        const uint64_t oh = f.u(64, 8);   // symbol-table message (0x11) of the root object header
        CN_REQUIRE(f.ok(oh, 16) && f.b[oh] == 1, CN_ERR_UNSUPPORTED, "cn_hdf5_read: %s: unsupported root object header", path);
        uint64_t p = oh + 16, end = p + f.u(oh + 8, 4);
        int left = (int)f.u(oh + 2, 2);
        while (left-- > 0 && f.ok(p, 8)) {
            const unsigned type = (unsigned)f.u(p, 2);
            const uint64_t size = f.u(p + 2, 2);
            if (type == 0x11 && f.ok(p + 8, 16)) { tree = f.u(p + 8, 8); heap = f.u(p + 16, 8); }
            p += 8 + size;
            if (p > end) break;
        }
    }
    CN_REQUIRE(tree && heap && f.ok(heap, 32) && memcmp(&f.b[heap], "HEAP", 4) == 0, CN_ERR_UNSUPPORTED,
               "cn_hdf5_read: %s: root group has no symbol table", path);
    const uint64_t heap_data = f.u(heap + 24, 8);
    const char *name = dataset[0] == '/' ? dataset + 1 : dataset;
    const uint64_t oh = h5_find(f, tree, heap_data, name, 0);
    CN_REQUIRE(oh && f.ok(oh, 16) && f.b[oh] == 1, CN_ERR_ARG, "cn_hdf5_read: dataset '%s' not found in %s", dataset, path);
    int left = (int)f.u(oh + 2, 2);
    const uint64_t hsize = f.u(oh + 8, 4);
    CN_REQUIRE(f.ok(oh + 16, hsize) && h5_parse_messages(f, oh + 16, oh + 16 + hsize, left, d, 0) && d.have_space && d.have_type && d.have_layout,
               CN_ERR_UNSUPPORTED, "cn_hdf5_read: dataset '%s' of %s uses a feature this reader does not have (chunking, big endian, rank > 2)", dataset, path);
    CN_REQUIRE(d.dims[0] < (1ull << 31) && d.dims[1] < (1ull << 31), CN_ERR_UNSUPPORTED, "cn_hdf5_read: dimension of 2^31 or more");
    n = d.dims[0] * (d.rank == 2 ? d.dims[1] : 1);
    CN_REQUIRE((d.type_class == 0 || d.type_class == 1) && (d.type_size == 4 || d.type_size == 8), CN_ERR_UNSUPPORTED,
               "cn_hdf5_read: datatype class %d size %d", d.type_class, d.type_size);
    CN_REQUIRE(n > 0 && n < (1ull << 40) && f.ok(d.data_addr, n * (uint64_t)d.type_size) && d.data_size >= n * (uint64_t)d.type_size,
               CN_ERR_ARG, "cn_hdf5_read: data of '%s' lies outside %s", dataset, path);
    return CN_OK;
}

// element i of the dataset converted to T the way H5Dread converts to a native type (value conversion, no scaling)
template <typename T>
void h5_convert(const H5 &f, const H5Dataset &d, uint64_t n, T *out)
{
    const unsigned char *src = &f.b[d.data_addr];
    for (uint64_t i = 0; i < n; ++i) {
        if (d.type_class == 1) {
            if (d.type_size == 4) { float v; memcpy(&v, src + 4 * i, 4); out[i] = (T)v; }
            else { double v; memcpy(&v, src + 8 * i, 8); out[i] = (T)v; }
        } else if (d.type_size == 4) {
            if (d.type_signed) { int32_t v; memcpy(&v, src + 4 * i, 4); out[i] = (T)v; }
            else { uint32_t v; memcpy(&v, src + 4 * i, 4); out[i] = (T)v; }
        } else {
            if (d.type_signed) { int64_t v; memcpy(&v, src + 8 * i, 8); out[i] = (T)v; }
            else { uint64_t v; memcpy(&v, src + 8 * i, 8); out[i] = (T)v; }
        }
    }
}

template <typename T>
int h5_read(const char *path, const char *dataset, T **data_out, int64_t *rows, int64_t *cols)
{
    CN_REQUIRE(path && dataset && data_out && rows && cols, CN_ERR_ARG, "cn_hdf5_read: null argument");
    *data_out = nullptr;
    H5 f;
    H5Dataset d;
    uint64_t n = 0;
    int st = h5_locate(path, dataset, f, d, n);
    if (st != CN_OK) return st;
    T *out = (T *)malloc(n * sizeof(T));
    CN_REQUIRE(out, CN_ERR_NOMEM, "cn_hdf5_read: out of memory");
    h5_convert(f, d, n, out);
    *data_out = out;
    *rows = (int64_t)d.dims[0];
    *cols = d.rank == 2 ? (int64_t)d.dims[1] : 1;
    return CN_OK;
}
}  // namespace

extern "C" int cn_hdf5_read_f32(const char *path, const char *dataset, float **data_out, int64_t *rows, int64_t *cols)
{
    return h5_read<float>(path, dataset, data_out, rows, cols);
}
// Shape alone, and conversion into a buffer of the caller (e.g. pinned memory), so that a large data set is neither
// allocated nor copied twice.
extern "C" int cn_hdf5_dims(const char *path, const char *dataset, int64_t *rows, int64_t *cols)
{
    CN_REQUIRE(path && dataset && rows && cols, CN_ERR_ARG, "cn_hdf5_dims: null argument");
    H5 f;
    H5Dataset d;
    uint64_t n = 0;
    int st = h5_locate(path, dataset, f, d, n);
    if (st != CN_OK) return st;
    *rows = (int64_t)d.dims[0];
    *cols = d.rank == 2 ? (int64_t)d.dims[1] : 1;
    return CN_OK;
}
extern "C" int cn_hdf5_read_f32_into(const char *path, const char *dataset, float *dst, int64_t capacity)
{
    CN_REQUIRE(path && dataset && dst && capacity >= 0, CN_ERR_ARG, "cn_hdf5_read_f32_into: bad argument");
    H5 f;
    H5Dataset d;
    uint64_t n = 0;
    int st = h5_locate(path, dataset, f, d, n);
    if (st != CN_OK) return st;
    CN_REQUIRE(n <= (uint64_t)capacity, CN_ERR_SHAPE, "cn_hdf5_read_f32_into: data set has %llu elements, the buffer %lld",
               (unsigned long long)n, (long long)capacity);
    h5_convert(f, d, n, dst);
    return CN_OK;
}
// the same for index data (the CSR files' /indices, /indptr, /shape): integers stay exact beyond 2^24
extern "C" int cn_hdf5_read_i32(const char *path, const char *dataset, int32_t **data_out, int64_t *rows, int64_t *cols)
{
    return h5_read<int32_t>(path, dataset, data_out, rows, cols);
}

extern "C" void cn_host_free(void *p) { free(p); }

// Writer for the same subset (write_hdf5, source/util.cu:202-216): one rank-2 float32 dataset, contiguous, in the
// root group of a version-0 file.  Block order and sizes follow what libhdf5 1.8 writes for such a file: superblock
// with the root symbol-table entry, root object header, group B-tree node (internal K = 16), local heap with its
// data segment, dataset object header, symbol-table node (leaf K = 4), data.
namespace {
struct H5Out {
    std::vector<unsigned char> b;
    void put(uint64_t v, int n) { for (int i = 0; i < n; ++i) b.push_back((unsigned char)(v >> (8 * i))); }
    void str(const char *s, size_t n) { b.insert(b.end(), s, s + n); }
    void pad_to(size_t off) { b.resize(off, 0); }
};
}  // namespace

extern "C" int cn_hdf5_write_f32(const char *path, const char *dataset, const float *data, int64_t rows, int64_t cols)
{
    CN_REQUIRE(path && dataset && data && rows > 0 && cols > 0, CN_ERR_ARG, "cn_hdf5_write_f32: bad argument");
    const char *name = dataset[0] == '/' ? dataset + 1 : dataset;
    const size_t nl = strlen(name);
    CN_REQUIRE(nl > 0 && nl < 64 && !strchr(name, '/'), CN_ERR_ARG, "cn_hdf5_write_f32: dataset name must be one path component shorter than 64 bytes");
    const uint64_t UNDEF = ~0ull;
    const uint64_t root_oh = 96, tree = 136, heap = 680, heap_data = 712, heap_size = 88, ds_oh = 800, snod = 928, data_addr = 2048;
    const uint64_t nbytes = (uint64_t)rows * (uint64_t)cols * 4;
    H5Out o;
    // superblock, version 0
    static const char sig[8] = {(char)0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};
    o.str(sig, 8);
    o.put(0, 1); o.put(0, 1); o.put(0, 1); o.put(0, 1); o.put(0, 1);   // versions: superblock, free space, root entry, -, shared header
    o.put(8, 1); o.put(8, 1); o.put(0, 1);                           // offset size, length size, -
    o.put(4, 2); o.put(16, 2); o.put(0, 4);                          // group leaf K, group internal K, consistency flags
    o.put(0, 8); o.put(UNDEF, 8); o.put(data_addr + nbytes, 8); o.put(UNDEF, 8);   // base, free-space info, end of file, driver info
    o.put(0, 8); o.put(root_oh, 8); o.put(1, 4); o.put(0, 4); o.put(tree, 8); o.put(heap, 8);   // root symbol-table entry
    // root object header: one symbol-table message
    o.pad_to(root_oh);
    o.put(1, 1); o.put(0, 1); o.put(1, 2); o.put(1, 4); o.put(24, 4); o.put(0, 4);
    o.put(0x11, 2); o.put(16, 2); o.put(0, 4); o.put(tree, 8); o.put(heap, 8);
    // group B-tree node, level 0, one child
    o.pad_to(tree);
    o.str("TREE", 4); o.put(0, 1); o.put(0, 1); o.put(1, 2); o.put(UNDEF, 8); o.put(UNDEF, 8);
    o.put(0, 8); o.put(snod, 8); o.put(8, 8);   // key 0 (empty name), child, key 1 (the dataset's name)
    // local heap: empty name at 0, the dataset's name at 8, the rest one free block
    o.pad_to(heap);
    const uint64_t name_end = 8 + ((nl + 1 + 7) & ~(size_t)7);
    CN_REQUIRE(name_end + 16 <= heap_size, CN_ERR_ARG, "cn_hdf5_write_f32: dataset name too long");
    o.str("HEAP", 4); o.put(0, 4); o.put(heap_size, 8); o.put(name_end, 8); o.put(heap_data, 8);
    o.pad_to(heap_data + 8);
    o.str(name, nl);
    o.pad_to(heap_data + name_end);
    o.put(1, 8); o.put(heap_size - name_end, 8);   // free block: no next block, its size
    // dataset object header: fill value, datatype (IEEE float32 little endian), dataspace, contiguous layout
    o.pad_to(ds_oh);
    o.put(1, 1); o.put(0, 1); o.put(4, 2); o.put(1, 4); o.put(16 + 32 + 32 + 32, 4); o.put(0, 4);
    o.put(0x5, 2); o.put(8, 2); o.put(1, 4); o.put(2, 1); o.put(2, 1); o.put(2, 1); o.put(1, 1); o.put(0, 4);
    o.put(0x3, 2); o.put(24, 2); o.put(1, 4);
    o.put(0x11, 1); o.put(0x20, 1); o.put(31, 1); o.put(0, 1); o.put(4, 4);
    o.put(0, 2); o.put(32, 2); o.put(23, 1); o.put(8, 1); o.put(0, 1); o.put(23, 1); o.put(127, 4); o.put(0, 4);
    o.put(0x1, 2); o.put(24, 2); o.put(0, 4);
    o.put(1, 1); o.put(2, 1); o.put(0, 1); o.put(0, 5); o.put((uint64_t)rows, 8); o.put((uint64_t)cols, 8);
    o.put(0x8, 2); o.put(24, 2); o.put(1, 4);
    o.put(3, 1); o.put(1, 1); o.put(data_addr, 8); o.put(nbytes, 8); o.put(0, 6);
    // symbol-table node: one entry
    o.pad_to(snod);
    o.str("SNOD", 4); o.put(1, 1); o.put(0, 1); o.put(1, 2);
    o.put(8, 8); o.put(ds_oh, 8); o.put(0, 4); o.put(0, 4); o.put(0, 8); o.put(0, 8);
    o.pad_to(data_addr);
    FILE *fp = fopen(path, "wb");
    CN_REQUIRE(fp, CN_ERR_ARG, "cn_hdf5_write_f32: cannot create %s", path);
    const bool ok = fwrite(o.b.data(), 1, o.b.size(), fp) == o.b.size() && fwrite(data, 1, nbytes, fp) == nbytes;
    const bool closed = fclose(fp) == 0;
    CN_REQUIRE(ok && closed, CN_ERR_ARG, "cn_hdf5_write_f32: short write to %s", path);
    return CN_OK;
}

// ------------------------------------------------------------------------------------------------
// Codebook file: dataset "/Default" (126 x 1 float32) of the reference's source/8bit_floats.hdf5, which the
// reference loads at source/clusterNet.cpp:73, or a raw 504-byte dump of the same table.
// ------------------------------------------------------------------------------------------------
extern "C" int cn_codebook_load(const char *path, float *tbl)
{
    CN_REQUIRE(path && tbl, CN_ERR_ARG, "cn_codebook_load: null argument");
    FILE *f = fopen(path, "rb");
    CN_REQUIRE(f, CN_ERR_ARG, "cn_codebook_load: cannot open %s", path);
    fseek(f, 0, SEEK_END);
    const long size = ftell(f);
    const long payload = CN_CODEBOOK_N * 4;
    if (size == payload) {
        fseek(f, 0, SEEK_SET);
        const size_t got = fread(tbl, 4, CN_CODEBOOK_N, f);
        fclose(f);
        CN_REQUIRE(got == CN_CODEBOOK_N, CN_ERR_ARG, "cn_codebook_load: short read from %s", path);
    } else {
        fclose(f);
        float *data = nullptr;
        int64_t rows = 0, cols = 0;
        int st = cn_hdf5_read_f32(path, "Default", &data, &rows, &cols);
        if (st != CN_OK) {
            std::string why = cn_last_error();
            cn_set_error("cn_codebook_load: %s is neither a 504-byte table nor a readable HDF5 file (%s)", path, why.c_str());
            return CN_ERR_ARG;
        }
        const bool shape_ok = rows * cols == CN_CODEBOOK_N;
        if (shape_ok) memcpy(tbl, data, payload);
        free(data);
        CN_REQUIRE(shape_ok, CN_ERR_ARG, "cn_codebook_load: /Default of %s has %lld x %lld entries, expected 126", path, (long long)rows, (long long)cols);
    }
    for (int i = 0; i < CN_CODEBOOK_N; ++i) {
        bool ok = tbl[i] > 0.f && tbl[i] < 1.f && (i == 0 || tbl[i] > tbl[i - 1]);
        CN_REQUIRE(ok, CN_ERR_ARG, "cn_codebook_load: entry %d of %s is not an increasing value in (0,1)", i, path);
    }
    return CN_OK;
}

// ------------------------------------------------------------------------------------------------
// Compressor decision function on a magnitude a = |x / precision| that is not NaN.
// Follows kCompression_8bit (source/clusterKernels.cu:1189-1229): two range tests, a six-step search
// that visits odd table indices starting at 63, then a nearest-of-two pick between the final (even)
// pivot and its lower neighbour.  Index 126 is outside the 126-entry table; the reference reads an
// unwritten shared-memory word there, this code takes it as +infinity (=> index 125 is chosen).
// ------------------------------------------------------------------------------------------------
static inline float tbl_at(const float *tbl, int i) { return i < CN_CODEBOOK_N ? tbl[i] : INFINITY; }

static uint8_t code_of_magnitude(const float *tbl, float a)
{
    const float threshold_lower = 0.0000015;
    const float threshold_upper = 0.995703;
    if (a < threshold_lower) return 254;
    if (a > threshold_upper) return 127;
    int pivot = 63, upper = 125, lower = 0;
    for (int j = 32; j > 0; j >>= 1) {
        if (a > tbl_at(tbl, pivot)) { lower = pivot; pivot += j; }
        else                        { upper = pivot; pivot -= j; }
    }
    float tp = tbl_at(tbl, pivot);
    if (lower == pivot) return (uint8_t)(fabsf(tp - a) < (tbl[upper] - a) ? pivot : upper);
    return (uint8_t)((tp - a) < fabsf(tbl[lower] - a) ? pivot : lower);
}

static inline int level_of_code(uint8_t c) { return c == 254 ? 0 : (c == 127 ? 127 : (int)c + 1); }

extern "C" int cn_codec_build_thresholds(const float *tbl, uint32_t *thr, uint8_t *level_codes)
{
    CN_REQUIRE(tbl && thr && level_codes, CN_ERR_ARG, "cn_codec_build_thresholds: null argument");
    for (int i = 0; i < CN_CODEBOOK_N; ++i) {
        bool ok = tbl[i] > 0.f && tbl[i] < 1.f && (i == 0 || tbl[i] > tbl[i - 1]);
        CN_REQUIRE(ok, CN_ERR_ARG, "codebook entry %d is not an increasing value in (0,1)", i);
    }
    level_codes[0] = 254;
    for (int i = 0; i < CN_CODEBOOK_N; ++i) level_codes[i + 1] = (uint8_t)i;
    level_codes[127] = 127;
    // The code is a non-decreasing step function of the magnitude (both rounded differences in the
    // pick move monotonically with a), so each level boundary is found by bisection on the ordered
    // fp32 bit patterns 0 .. +inf.
    for (int j = 1; j <= CN_NUM_THR; ++j) {
        uint32_t lo = 0, hi = 0x7f800000u;
        while (lo < hi) {
            uint32_t mid = lo + ((hi - lo) >> 1);
            float a;
            memcpy(&a, &mid, 4);
            if (level_of_code(code_of_magnitude(tbl, a)) >= j) hi = mid; else lo = mid + 1;
        }
        thr[j - 1] = lo;
    }
    // Spot-check the bisection's premise on both sides of every boundary and on the table values.
    for (int j = 0; j < CN_NUM_THR; ++j) {
        for (int d = -2; d <= 2; ++d) {
            int64_t ub = (int64_t)thr[j] + d;
            if (ub < 0 || ub > 0x7f800000LL) continue;
            uint32_t u = (uint32_t)ub;
            float a;
            memcpy(&a, &u, 4);
            int cnt = 0;
            for (int k = 0; k < CN_NUM_THR; ++k) cnt += thr[k] <= u;
            CN_REQUIRE(level_codes[cnt] == code_of_magnitude(tbl, a), CN_ERR_UNSUPPORTED,
                       "codebook yields a non-monotone decision function near threshold %d", j);
        }
    }
    return CN_OK;
}

// ------------------------------------------------------------------------------------------------
extern "C" int cn_context_create(int device, const float *codebook, cn_context **out)
{
    CN_REQUIRE(out && codebook, CN_ERR_ARG, "cn_context_create: null argument");
    *out = nullptr;
    int ndev = 0;
    CN_CUDA(cudaGetDeviceCount(&ndev));
    CN_REQUIRE(device >= 0 && device < ndev, CN_ERR_ARG, "cn_context_create: device %d of %d", device, ndev);
    CN_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    CN_CUDA(cudaGetDeviceProperties(&prop, device));
    CN_REQUIRE(prop.major == 10, CN_ERR_UNSUPPORTED,
               "this library holds sm_100a code only; device %d is sm_%d%d", device, prop.major, prop.minor);
    cn_context *c = new cn_context();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    memcpy(c->h_tbl, codebook, CN_CODEBOOK_N * sizeof(float));
    c->h_tbl[126] = INFINITY;
    c->h_tbl[127] = INFINITY;
    int st = cn_codec_build_thresholds(codebook, c->h_thr, c->h_level_codes);
    if (st != CN_OK) { delete c; return st; }
    c->h_thr[127] = 0xffffffffu;
    cudaError_t e;
    if ((e = cudaMalloc(&c->d_tbl, 128 * sizeof(float))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_thr, 128 * sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_level_codes, 128)) != cudaSuccess ||
        (e = cudaMalloc(&c->d_partials, CN_MAX_PARTIALS * sizeof(float))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_ticket, 64)) != cudaSuccess ||
        (e = cudaMemcpy(c->d_tbl, c->h_tbl, 128 * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(c->d_thr, c->h_thr, 128 * sizeof(uint32_t), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(c->d_level_codes, c->h_level_codes, 128, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemset(c->d_ticket, 0, 64)) != cudaSuccess) {
        cn_context_destroy(c);
        return cn_cuda_fail(e, "cn_context_create");
    }
    *out = c;
    return CN_OK;
}

extern "C" int cn_context_destroy(cn_context *c)
{
    if (!c) return CN_OK;
    cudaSetDevice(c->device);
    cn_comm_state_free(c);
    cn_gemm_workspace_free(c);
    for (auto &kv : c->timers) {
        if (kv.second.start) cudaEventDestroy(kv.second.start);
        if (kv.second.stop) cudaEventDestroy(kv.second.stop);
    }
    cudaFree(c->d_tbl);
    cudaFree(c->d_thr);
    cudaFree(c->d_level_codes);
    cudaFree(c->d_partials);
    cudaFree(c->d_ticket);
    delete c;
    return CN_OK;
}

extern "C" int cn_context_device(const cn_context *c) { return c ? c->device : -1; }

// ------------------------------------------------------------------------------------------------
// Named cumulative timers (ClusterNet::tick / tock, source/clusterNet.cpp:798-840): tick records a
// start event on the stream; tock records the stop event, waits for it and adds the elapsed
// milliseconds to the named total, which it returns.
// ------------------------------------------------------------------------------------------------
extern "C" int cn_tick(cn_context *c, const char *name, void *stream)
{
    CN_REQUIRE(c && name, CN_ERR_ARG, "cn_tick: null argument");
    cn_timer_slot &t = c->timers[name];
    if (!t.start) {
        CN_CUDA(cudaEventCreate(&t.start));
        CN_CUDA(cudaEventCreate(&t.stop));
    }
    CN_CUDA(cudaEventRecord(t.start, cn_stream(stream)));
    return CN_OK;
}

extern "C" int cn_tock(cn_context *c, const char *name, void *stream, float *cumulative_ms)
{
    CN_REQUIRE(c && name, CN_ERR_ARG, "cn_tock: null argument");
    auto it = c->timers.find(name);
    CN_REQUIRE(it != c->timers.end() && it->second.start, CN_ERR_ARG, "cn_tock: no tick for '%s'", name);
    cn_timer_slot &t = it->second;
    CN_CUDA(cudaEventRecord(t.stop, cn_stream(stream)));
    CN_CUDA(cudaEventSynchronize(t.stop));
    float ms = 0.f;
    CN_CUDA(cudaEventElapsedTime(&ms, t.start, t.stop));
    t.cumulative_ms += ms;
    if (cumulative_ms) *cumulative_ms = t.cumulative_ms;
    return CN_OK;
}
