// Minimal .npz reader for the expert weight file.
//
// Accepts what the reference's patched cnpy accepts (plugin/thirdparty/cnpy/cnpy.cpp:229-276,
// header parsing :109-156): zip local file headers walked sequentially until the
// central directory, compression method 0 (stored) or 8 (deflate), ".npy"
// stripped from member names, npy header v1/v2 with little-endian '<f4' data.
// The member size is taken from the npy header, so numpy's zip64 local headers
// (sizes 0xFFFFFFFF plus an extra field) work for stored members.
//
// Like cnpy, the `fortran_order` flag of a member is NOT honoured: the bytes are
// taken as a C-ordered array of the stated shape (cnpy.cpp:118-123 parses the
// flag and drops it).  The reference's own generator writes `wo_weight` that
// way (python/infmoe/config.py:52), so honouring the flag would change results
// relative to the reference.  A warning is printed once per file.
#include "npz.h"

#include <fcntl.h>
#include <unistd.h>
#include <zlib.h>

#include <atomic>
#include <cstdio>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"

namespace infmoe {

namespace {

struct File {
    FILE* f = nullptr;
    ~File() {
        if (f) fclose(f);
    }
};

bool read_exact(FILE* f, void* dst, size_t n) { return fread(dst, 1, n, f) == n; }

uint16_t le16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
uint32_t le32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

// Parses "{'descr': '<f4', 'fortran_order': False, 'shape': (3, 4), }"
int parse_npy_dict(const std::string& h, std::string& descr, bool& fortran, std::vector<int64_t>& shape) {
    size_t p = h.find("'descr'");
    if (p == std::string::npos) return INFMOE_ERR_FORMAT;
    p = h.find('\'', p + 7);
    if (p == std::string::npos) return INFMOE_ERR_FORMAT;
    size_t q = h.find('\'', p + 1);
    if (q == std::string::npos) return INFMOE_ERR_FORMAT;
    descr = h.substr(p + 1, q - p - 1);
    p = h.find("'fortran_order'");
    if (p == std::string::npos) return INFMOE_ERR_FORMAT;
    p = h.find(':', p);
    if (p == std::string::npos) return INFMOE_ERR_FORMAT;
    const size_t v = h.find_first_not_of(" ", p + 1);
    if (v == std::string::npos) return INFMOE_ERR_FORMAT;
    fortran = h.compare(v, 4, "True") == 0;
    p = h.find("'shape'");
    if (p == std::string::npos) return INFMOE_ERR_FORMAT;
    p = h.find('(', p);
    q = h.find(')', p);
    if (p == std::string::npos || q == std::string::npos) return INFMOE_ERR_FORMAT;
    shape.clear();
    int64_t cur = -1;
    for (size_t i = p + 1; i < q; ++i) {
        const char c = h[i];
        if (c >= '0' && c <= '9') {
            cur = (cur < 0 ? 0 : cur) * 10 + (c - '0');
        } else if (cur >= 0) {
            shape.push_back(cur);
            cur = -1;
        }
    }
    if (cur >= 0) shape.push_back(cur);
    return INFMOE_OK;
}

// Source of member bytes: either the file itself (stored) or an inflate stream over it.
class Member {
  public:
    Member(FILE* f, bool deflated, uint64_t comp_size) : f_(f), deflated_(deflated), comp_left_(comp_size) {
        if (deflated_) {
            memset(&z_, 0, sizeof(z_));
            ok_ = inflateInit2(&z_, -MAX_WBITS) == Z_OK;
            buf_.resize(1 << 20);
        }
    }
    ~Member() {
        if (deflated_ && ok_) inflateEnd(&z_);
    }
    bool read(void* dst, size_t n) {
        if (!deflated_) return read_exact(f_, dst, n);
        if (!ok_) return false;
        z_.next_out = (Bytef*)dst;
        size_t done = 0;
        while (done < n) {
            const size_t want = n - done < (1u << 30) ? n - done : (1u << 30);
            z_.avail_out = (uInt)want;
            if (z_.avail_in == 0) {
                size_t chunk = buf_.size();
                if (comp_left_ < chunk) chunk = (size_t)comp_left_;
                if (chunk == 0) return false;
                if (!read_exact(f_, buf_.data(), chunk)) return false;
                comp_left_ -= chunk;
                z_.next_in = buf_.data();
                z_.avail_in = (uInt)chunk;
            }
            const int rc = inflate(&z_, Z_NO_FLUSH);
            done += want - z_.avail_out;
            if (rc == Z_STREAM_END) break;
            if (rc != Z_OK) return false;
        }
        return done == n;
    }
    // Skips whatever compressed bytes of this member were not consumed.
    bool finish() {
        if (!deflated_) return true;
        return comp_left_ == 0 || fseeko(f_, (off_t)comp_left_, SEEK_CUR) == 0;
    }

  private:
    FILE* f_;
    bool deflated_;
    uint64_t comp_left_;
    z_stream z_;
    bool ok_ = true;
    std::vector<uint8_t> buf_;
};

// One member whose data is read after the walk, by a worker thread with a file descriptor of its own.
struct Job {
    std::string name;
    bool deflated = false;
    uint64_t offset = 0;       // stored: first payload byte; deflated: first byte of the compressed stream
    uint64_t comp_size = 0;    // deflated: compressed bytes
    size_t skip = 0;           // deflated: uncompressed bytes before the payload (the npy header)
    size_t bytes = 0;          // payload bytes
    float* dst = nullptr;
};

bool pread_exact(int fd, void* dst, size_t n, uint64_t off) {
    uint8_t* p = (uint8_t*)dst;
    while (n) {
        const ssize_t got = pread(fd, p, n < (1u << 30) ? n : (1u << 30), (off_t)off);
        if (got <= 0) return false;
        p += got;
        off += (uint64_t)got;
        n -= (size_t)got;
    }
    return true;
}

bool run_job(int fd, const Job& j) {
    if (!j.deflated) return pread_exact(fd, j.dst, j.bytes, j.offset);
    z_stream z;
    memset(&z, 0, sizeof(z));
    if (inflateInit2(&z, -MAX_WBITS) != Z_OK) return false;
    std::vector<uint8_t> in(1 << 20), head(j.skip ? j.skip : 1);
    uint64_t off = j.offset, left = j.comp_size;
    bool ok = true;
    // two output segments: the npy header (discarded), then the payload
    for (int seg = 0; seg < 2 && ok; ++seg) {
        uint8_t* out = seg == 0 ? head.data() : (uint8_t*)j.dst;
        size_t want = seg == 0 ? j.skip : j.bytes, done = 0;
        while (done < want) {
            if (z.avail_in == 0) {
                const size_t chunk = left < in.size() ? (size_t)left : in.size();
                if (chunk == 0 || !pread_exact(fd, in.data(), chunk, off)) { ok = false; break; }
                off += chunk;
                left -= chunk;
                z.next_in = in.data();
                z.avail_in = (uInt)chunk;
            }
            const size_t room = want - done < (1u << 30) ? want - done : (1u << 30);
            z.next_out = out + done;
            z.avail_out = (uInt)room;
            const int rc = inflate(&z, Z_NO_FLUSH);
            done += room - z.avail_out;
            if (rc == Z_STREAM_END) break;
            if (rc != Z_OK) { ok = false; break; }
        }
        ok = ok && done == want;
    }
    inflateEnd(&z);
    return ok;
}

}  // namespace

int npz_read(const char* path, const NpzAllocFn& alloc, bool* saw_fortran_order, int threads) {
    std::vector<Job> jobs;
    const bool deferred = threads > 1;
    File file;
    file.f = fopen(path, "rb");
    if (!file.f) {
        set_error("cannot open weight file %s", path);
        return INFMOE_ERR_IO;
    }
    bool warned = false;
    if (saw_fortran_order) *saw_fortran_order = false;
    while (true) {
        uint8_t lh[30];
        if (!read_exact(file.f, lh, 30)) {
            set_error("%s: truncated zip local header", path);
            return INFMOE_ERR_FORMAT;
        }
        if (!(lh[0] == 'P' && lh[1] == 'K')) {
            set_error("%s: not a zip/npz file", path);
            return INFMOE_ERR_FORMAT;
        }
        if (lh[2] != 0x03 || lh[3] != 0x04) break;  // central directory (or end record): all members read
        const uint16_t flags = le16(lh + 6), method = le16(lh + 8);
        uint64_t comp_size = le32(lh + 18);
        const uint16_t name_len = le16(lh + 26), extra_len = le16(lh + 28);
        std::string name(name_len, '\0');
        std::vector<uint8_t> extra(extra_len);
        if (!read_exact(file.f, &name[0], name_len) || (extra_len && !read_exact(file.f, extra.data(), extra_len))) {
            set_error("%s: truncated zip member header", path);
            return INFMOE_ERR_FORMAT;
        }
        if (comp_size == 0xFFFFFFFFu) {  // zip64 extra field 0x0001: uncompressed size, compressed size
            for (size_t i = 0; i + 4 <= extra.size();) {
                const uint16_t id = le16(&extra[i]), sz = le16(&extra[i + 2]);
                if (id == 0x0001 && sz >= 16 && i + 4 + 16 <= extra.size()) {
                    comp_size = 0;
                    for (int b = 7; b >= 0; --b) comp_size = (comp_size << 8) | extra[i + 4 + 8 + b];
                }
                i += 4 + (size_t)sz;
            }
        }
        if (method != 0 && method != 8) {
            set_error("%s: member %s uses unsupported compression method %d", path, name.c_str(), (int)method);
            return INFMOE_ERR_FORMAT;
        }
        if (method == 8 && (flags & 8)) {
            set_error("%s: member %s is deflated with a streamed size (data descriptor); not supported", path,
                      name.c_str());
            return INFMOE_ERR_FORMAT;
        }
        if (name.size() > 4 && name.compare(name.size() - 4, 4, ".npy") == 0) name.resize(name.size() - 4);

        const uint64_t member_start = (uint64_t)ftello(file.f);
        Member m(file.f, method == 8, comp_size);
        uint8_t pre[10];
        if (!m.read(pre, 10) || memcmp(pre, "\x93NUMPY", 6) != 0) {
            set_error("%s: member %s is not an npy array", path, name.c_str());
            return INFMOE_ERR_FORMAT;
        }
        size_t hlen = le16(pre + 8);
        std::string header;
        if (pre[6] >= 2) {  // v2/v3: 4-byte header length
            uint8_t more[2];
            if (!m.read(more, 2)) return INFMOE_ERR_FORMAT;
            hlen |= (size_t)le16(more) << 16;
        }
        header.resize(hlen);
        if (!m.read(&header[0], hlen)) {
            set_error("%s: member %s has a truncated npy header", path, name.c_str());
            return INFMOE_ERR_FORMAT;
        }
        std::string descr;
        bool fortran = false;
        std::vector<int64_t> shape;
        if (parse_npy_dict(header, descr, fortran, shape) != INFMOE_OK) {
            set_error("%s: member %s has a malformed npy header", path, name.c_str());
            return INFMOE_ERR_FORMAT;
        }
        if (descr != "<f4" && descr != "|f4" && descr != "=f4") {
            set_error("%s: member %s has dtype %s, expected little-endian float32", path, name.c_str(), descr.c_str());
            return INFMOE_ERR_FORMAT;
        }
        if (fortran) {
            if (saw_fortran_order) *saw_fortran_order = true;
            if (!warned) {
                fprintf(stderr,
                        "WARNING: %s: member %s is flagged fortran_order; like the reference reader the bytes are "
                        "taken as C order\n",
                        path, name.c_str());
                warned = true;
            }
        }
        size_t count = 1;
        for (int64_t d : shape) {
            if (d < 0 || (d > 0 && count > (SIZE_MAX / sizeof(float)) / (size_t)d)) {
                set_error("%s: member %s has a shape whose element count overflows", path, name.c_str());
                return INFMOE_ERR_FORMAT;
            }
            count *= (size_t)d;
        }
        float* dst = nullptr;
        const int rc = alloc(name, shape, &dst);
        if (rc != INFMOE_OK) return rc;
        if (dst && deferred) {
            Job j;
            j.name = name;
            j.deflated = method == 8;
            j.offset = j.deflated ? member_start : (uint64_t)ftello(file.f);
            j.comp_size = comp_size;
            j.skip = (pre[6] >= 2 ? 12 : 10) + hlen;
            j.bytes = count * sizeof(float);
            j.dst = dst;
            jobs.push_back(j);
            if (method == 0 && fseeko(file.f, (off_t)(count * sizeof(float)), SEEK_CUR) != 0) return INFMOE_ERR_IO;
        } else if (dst) {
            if (!m.read(dst, count * sizeof(float))) {
                set_error("%s: member %s is truncated", path, name.c_str());
                return INFMOE_ERR_FORMAT;
            }
        } else if (method == 0) {
            if (fseeko(file.f, (off_t)(count * sizeof(float)), SEEK_CUR) != 0) return INFMOE_ERR_IO;
        }
        if (!m.finish()) return INFMOE_ERR_IO;
        if (method == 0 && (flags & 8)) {
            // stored with a trailing data descriptor: optional signature + crc + sizes (32- or 64-bit)
            uint8_t dd[4];
            if (!read_exact(file.f, dd, 4)) return INFMOE_ERR_FORMAT;
            const bool sig = le32(dd) == 0x08074b50u;
            const size_t rest = (sig ? 4 : 0) + (comp_size > 0xFFFFFFFEull ? 16 : 8);
            if (fseeko(file.f, (off_t)rest, SEEK_CUR) != 0) return INFMOE_ERR_IO;
        }
    }
    if (jobs.empty()) return INFMOE_OK;
    // The members' data, read (and inflated) by a few threads at once: every member is an independent range of
    // the file, and one thread neither saturates the storage nor, for deflated files, the decompressor.
    const int n = (int)jobs.size() < threads ? (int)jobs.size() : threads;
    std::atomic<size_t> next{0};
    std::atomic<int> failed{-1};
    auto worker = [&]() {
        const int fd = open(path, O_RDONLY);
        if (fd < 0) {
            failed.store((int)jobs.size());
            return;
        }
        for (size_t i; (i = next.fetch_add(1)) < jobs.size() && failed.load() < 0;)
            if (!run_job(fd, jobs[i])) failed.store((int)i);
        close(fd);
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < n; ++t) pool.emplace_back(worker);
    worker();
    for (auto& t : pool) t.join();
    const int bad = failed.load();
    if (bad >= 0) {
        if (bad >= (int)jobs.size()) set_error("cannot open weight file %s", path);
        else set_error("%s: member %s is truncated or corrupt", path, jobs[(size_t)bad].name.c_str());
        return bad >= (int)jobs.size() ? INFMOE_ERR_IO : INFMOE_ERR_FORMAT;
    }
    return INFMOE_OK;
}

}  // namespace infmoe
