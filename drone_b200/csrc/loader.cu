// Loading partitions from disk (host code).
//
// 1. The reference's text formats — G.<p> ("u v" per line), Master.<p> ("vertex worker worker ..." per line),
//    Mirror.<p> ("vertex worker" per line) — are read there with fscanf / getline / istringstream loops
//    (cuda_gcn/src/common/parser.cu:72-131) and with bufio + strings.Split in the Go loader
//    (DRONE/src/graph/cuda_graph.go:32-60), one token at a time on one core.  Here a file is mapped once and parsed by
//    all host threads: the file is cut at line ends, every thread counts the integers and lines of its piece, a prefix
//    sum gives every piece its place in the output, and a second pass writes the values.
// 2. A binary format for a whole partition (edges of all parts, owner / replica tables, one presence word per vertex)
//    from which a rank reads its own edges and the global tables with two preads — no parsing, no renumbering of what
//    it does not hold.  The reference has no counterpart.
#include "common.cuh"

#include <algorithm>
#include <cerrno>
#include <cstdint>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace drone {

struct MappedFile {
    const char *data = nullptr;
    size_t size = 0;
    int fd = -1;
    ~MappedFile() {
        if (data && size) munmap(const_cast<char *>(data), size);
        if (fd >= 0) close(fd);
    }
};

static int map_file(const char *path, MappedFile &m) {
    m.fd = open(path, O_RDONLY);
    if (m.fd < 0) return set_error(DRONE_E_INVALID, "cannot open %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(m.fd, &st) != 0) return set_error(DRONE_E_INVALID, "cannot stat %s: %s", path, strerror(errno));
    m.size = (size_t)st.st_size;
    if (m.size == 0) return DRONE_OK;
    void *p = mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, m.fd, 0);
    if (p == MAP_FAILED) {
        m.size = 0;
        return set_error(DRONE_E_INVALID, "cannot map %s: %s", path, strerror(errno));
    }
    m.data = (const char *)p;
    madvise(p, m.size, MADV_SEQUENTIAL);
    return DRONE_OK;
}

// Pieces of the file that start right after a line end (or at 0).
static std::vector<size_t> cut_at_lines(const MappedFile &m, int pieces) {
    std::vector<size_t> cut{0};
    for (int i = 1; i < pieces; ++i) {
        size_t at = m.size / pieces * i;
        if (at <= cut.back()) continue;
        while (at < m.size && m.data[at - 1] != '\n') ++at;
        if (at > cut.back() && at < m.size) cut.push_back(at);
    }
    cut.push_back(m.size);
    return cut;
}

// One pass over [b, e): counts (values == NULL) or writes.  Lines without an integer are skipped.
// Returns the offset of the first byte that is neither a digit, a sign, nor white space, or -1.
// With `odd` set the values are dealt out in turn: value k of the file goes to values[k / 2] (k even) or odd[k / 2].
static long long scan_piece(const char *d, size_t b, size_t e, long long *n_values, long long *n_lines, int *values,
                            long long *line_start, long long value_base, int *odd = nullptr) {
    long long nv = 0, nl = 0;
    bool line_has_value = false;
    size_t i = b;
    while (i < e) {
        const char c = d[i];
        if (c == '\n') {
            line_has_value = false;
            ++i;
        } else if (c == ' ' || c == '\t' || c == '\r') {
            ++i;
        } else if ((c >= '0' && c <= '9') || c == '-' || c == '+') {
            bool neg = false;
            if (c == '-' || c == '+') {
                neg = c == '-';
                ++i;
                if (i >= e || d[i] < '0' || d[i] > '9') return (long long)i;
            }
            long long x = 0;
            while (i < e && d[i] >= '0' && d[i] <= '9') {
                x = x * 10 + (d[i] - '0');
                if (x > 2147483648LL) return (long long)i;
                ++i;
            }
            if (neg) x = -x;
            if (x > 2147483647LL) return (long long)i;
            if (!line_has_value) {
                if (line_start) line_start[nl] = value_base + nv;
                ++nl;
                line_has_value = true;
            }
            if (odd) {
                const long long k = value_base + nv;
                ((k & 1) ? odd : values)[k >> 1] = (int)x;
            } else if (values) {
                values[nv] = (int)x;
            }
            ++nv;
        } else {
            return (long long)i;
        }
    }
    *n_values = nv;
    *n_lines = nl;
    return -1;
}

static int parse_text(const char *path, long long *n_values, long long *n_lines, int *values, long long cap_values,
                      long long *line_start, long long cap_lines, int *odd = nullptr) {
    MappedFile m;
    int rc = map_file(path, m);
    if (rc) return rc;
    int threads = (int)std::thread::hardware_concurrency();
    if (threads < 1) threads = 1;
    if (m.size < (1u << 20)) threads = 1;
    const std::vector<size_t> cut = cut_at_lines(m, threads);
    const int P = (int)cut.size() - 1;
    std::vector<long long> nv(P, 0), nl(P, 0), bad(P, -1);
    auto run = [&](bool write, const std::vector<long long> &vbase, const std::vector<long long> &lbase) {
        std::vector<std::thread> pool;
        for (int p = 0; p < P; ++p)
            pool.emplace_back([&, p] {
                long long a = 0, b = 0;
                int *out = !write ? nullptr : (odd ? values : values + vbase[p]);   // dealt output is indexed globally
                bad[p] = scan_piece(m.data, cut[p], cut[p + 1], &a, &b, out,
                                    write && line_start ? line_start + lbase[p] : nullptr, write ? vbase[p] : 0,
                                    write ? odd : nullptr);
                nv[p] = a;
                nl[p] = b;
            });
        for (auto &t : pool) t.join();
    };
    std::vector<long long> vbase(P + 1, 0), lbase(P + 1, 0);
    run(false, vbase, lbase);
    for (int p = 0; p < P; ++p) {
        if (bad[p] >= 0) return set_error(DRONE_E_INVALID, "%s: byte %lld is not part of an integer that fits 32 bits", path, bad[p]);
        vbase[p + 1] = vbase[p] + nv[p];
        lbase[p + 1] = lbase[p] + nl[p];
    }
    *n_values = vbase[P];
    *n_lines = lbase[P];
    if (!values) return DRONE_OK;
    if (cap_values < vbase[P] || (line_start && cap_lines < lbase[P]))
        return set_error(DRONE_E_INVALID, "%s holds %lld integers on %lld lines, the buffers hold %lld / %lld", path, vbase[P],
                         lbase[P], cap_values, cap_lines);
    run(true, vbase, lbase);
    if (line_start) line_start[lbase[P]] = vbase[P];
    return DRONE_OK;
}

static const char kMagic[8] = {'D', 'R', 'N', 'P', 'A', 'R', 'T', '1'};

struct PartitionHeader {
    char magic[8];
    int32_t n_vertices, n_parts;
    int64_t n_edges;
};

static int write_all(int fd, const void *p, size_t n, const char *path) {
    const char *c = (const char *)p;
    while (n > 0) {
        const ssize_t w = write(fd, c, std::min<size_t>(n, (size_t)1 << 30));
        if (w <= 0) return set_error(DRONE_E_INVALID, "write to %s failed: %s", path, strerror(errno));
        c += w;
        n -= (size_t)w;
    }
    return DRONE_OK;
}

static int read_at(int fd, void *p, size_t n, off_t at, const char *path) {
    char *c = (char *)p;
    while (n > 0) {
        const ssize_t r = pread(fd, c, std::min<size_t>(n, (size_t)1 << 30), at);
        if (r <= 0) return set_error(DRONE_E_INVALID, "%s is shorter than its header says", path);
        c += r;
        at += r;
        n -= (size_t)r;
    }
    return DRONE_OK;
}

struct Fd {
    int fd = -1;
    ~Fd() { if (fd >= 0) close(fd); }
};

static int open_partition(const char *path, Fd &f, PartitionHeader &h, std::vector<long long> &off) {
    f.fd = open(path, O_RDONLY);
    if (f.fd < 0) return set_error(DRONE_E_INVALID, "cannot open %s: %s", path, strerror(errno));
    int rc = read_at(f.fd, &h, sizeof(h), 0, path);
    if (rc) return rc;
    if (memcmp(h.magic, kMagic, 8) != 0) return set_error(DRONE_E_INVALID, "%s is not a partition file (bad magic)", path);
    if (h.n_vertices <= 0 || h.n_parts < 1 || h.n_parts > 64 || h.n_edges < 0)
        return set_error(DRONE_E_INVALID, "%s: implausible header (V=%d, parts=%d, E=%lld)", path, h.n_vertices, h.n_parts,
                         (long long)h.n_edges);
    off.resize((size_t)h.n_parts + 1);
    rc = read_at(f.fd, off.data(), sizeof(long long) * off.size(), sizeof(h), path);
    if (rc) return rc;
    if (off[0] != 0 || off[h.n_parts] != h.n_edges) return set_error(DRONE_E_INVALID, "%s: part offsets do not add up", path);
    for (int p = 0; p < h.n_parts; ++p)
        if (off[p + 1] < off[p]) return set_error(DRONE_E_INVALID, "%s: part offsets decrease", path);
    return DRONE_OK;
}

}  // namespace drone

using namespace drone;

extern "C" {

int drone_text_ints_count(const char *path, long long *n_values, long long *n_lines) {
    DRONE_REQUIRE(path && n_values && n_lines, "drone_text_ints_count: NULL argument");
    return parse_text(path, n_values, n_lines, nullptr, 0, nullptr, 0);
}

int drone_text_ints_read(const char *path, int *values, long long cap_values, long long *line_start, long long cap_lines,
                         long long *n_values, long long *n_lines) {
    DRONE_REQUIRE(path && values, "drone_text_ints_read: NULL argument");
    long long nv = 0, nl = 0;
    const int rc = parse_text(path, &nv, &nl, values, cap_values, line_start, cap_lines);
    if (n_values) *n_values = nv;
    if (n_lines) *n_lines = nl;
    return rc;
}

int drone_text_edges_read(const char *path, int *u, int *v, long long cap_edges, long long *n_edges) {
    DRONE_REQUIRE(path && u && v && n_edges, "drone_text_edges_read: NULL argument");
    long long nv = 0, nl = 0;
    const int rc = parse_text(path, &nv, &nl, u, 2 * cap_edges, nullptr, 0, v);
    if (rc) return rc;
    if (nv & 1) return set_error(DRONE_E_INVALID, "%s holds an odd number of integers (%lld)", path, nv);
    *n_edges = nv / 2;
    return DRONE_OK;
}

int drone_partition_write(const char *path, int n_vertices, int n_parts, const long long *part_offset, const int *u,
                          const int *v, const int *owner, const int *replicas, const unsigned long long *present_bits) {
    DRONE_REQUIRE(path && part_offset && owner && replicas && present_bits, "drone_partition_write: NULL argument");
    DRONE_REQUIRE(n_vertices > 0 && n_parts >= 1 && n_parts <= 64, "drone_partition_write: bad sizes (V=%d, parts=%d)", n_vertices,
                  n_parts);
    const long long e = part_offset[n_parts];
    DRONE_REQUIRE(part_offset[0] == 0 && e >= 0 && (e == 0 || (u && v)), "drone_partition_write: bad edge arrays");
    Fd f;
    f.fd = open(path, O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (f.fd < 0) return set_error(DRONE_E_INVALID, "cannot create %s: %s", path, strerror(errno));
    PartitionHeader h;
    memcpy(h.magic, kMagic, 8);
    h.n_vertices = n_vertices;
    h.n_parts = n_parts;
    h.n_edges = e;
    int rc;
    if ((rc = write_all(f.fd, &h, sizeof(h), path))) return rc;
    if ((rc = write_all(f.fd, part_offset, sizeof(long long) * ((size_t)n_parts + 1), path))) return rc;
    if ((rc = write_all(f.fd, owner, sizeof(int) * (size_t)n_vertices, path))) return rc;
    if ((rc = write_all(f.fd, replicas, sizeof(int) * (size_t)n_vertices, path))) return rc;
    if ((rc = write_all(f.fd, present_bits, sizeof(unsigned long long) * (size_t)n_vertices, path))) return rc;
    if ((rc = write_all(f.fd, u, sizeof(int) * (size_t)e, path))) return rc;
    if ((rc = write_all(f.fd, v, sizeof(int) * (size_t)e, path))) return rc;
    return DRONE_OK;
}

int drone_partition_read_header(const char *path, int *n_vertices, int *n_parts, long long *part_offset) {
    DRONE_REQUIRE(path && n_vertices && n_parts && part_offset, "drone_partition_read_header: NULL argument");
    Fd f;
    PartitionHeader h;
    std::vector<long long> off;
    const int rc = open_partition(path, f, h, off);
    if (rc) return rc;
    *n_vertices = h.n_vertices;
    *n_parts = h.n_parts;
    std::copy(off.begin(), off.end(), part_offset);
    return DRONE_OK;
}

int drone_partition_read(const char *path, int part, int *u, int *v, int *owner, int *replicas,
                         unsigned long long *present_bits) {
    DRONE_REQUIRE(path != nullptr, "drone_partition_read: NULL path");
    Fd f;
    PartitionHeader h;
    std::vector<long long> off;
    int rc = open_partition(path, f, h, off);
    if (rc) return rc;
    DRONE_REQUIRE(part >= -1 && part < h.n_parts, "drone_partition_read: part %d of %d", part, h.n_parts);
    const size_t V = (size_t)h.n_vertices;
    off_t at = (off_t)(sizeof(h) + sizeof(long long) * off.size());
    if (owner && (rc = read_at(f.fd, owner, sizeof(int) * V, at, path))) return rc;
    at += (off_t)(sizeof(int) * V);
    if (replicas && (rc = read_at(f.fd, replicas, sizeof(int) * V, at, path))) return rc;
    at += (off_t)(sizeof(int) * V);
    if (present_bits && (rc = read_at(f.fd, present_bits, sizeof(unsigned long long) * V, at, path))) return rc;
    at += (off_t)(sizeof(unsigned long long) * V);
    const long long e0 = part < 0 ? 0 : off[part], e1 = part < 0 ? h.n_edges : off[part + 1];
    const size_t bytes = sizeof(int) * (size_t)(e1 - e0);
    if (u && bytes && (rc = read_at(f.fd, u, bytes, at + (off_t)(sizeof(int) * (size_t)e0), path))) return rc;
    at += (off_t)(sizeof(int) * (size_t)h.n_edges);
    if (v && bytes && (rc = read_at(f.fd, v, bytes, at + (off_t)(sizeof(int) * (size_t)e0), path))) return rc;
    return DRONE_OK;
}

}  // extern "C"
