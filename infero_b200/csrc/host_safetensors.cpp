// Reader of the safetensors container (host only): the file is mapped read-only, its JSON header is
// parsed and checked here, and tensors are handed out as (dtype, shape, pointer into the mapping).
//
// File = 8-byte little-endian header length, a JSON object mapping each tensor name to
// {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to the end of the header; an
// optional "__metadata__" object of strings), then the raw little-endian payload.  The checks
// mirror the reference's (crates/safetensors/src/lib.rs:390-436): header inside the file, offsets
// inside the payload, byte count == prod(shape) * element size, known dtypes only (:47-58).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Tensor {
    std::string name;
    int dtype = 0;                       // index into DTYPES
    std::vector<long long> shape;
    long long begin = 0, nbytes = 0;     // begin: offset in the file
};

struct File {
    std::string path, error;
    int fd = -1;
    void* map = nullptr;
    size_t size = 0;
    std::vector<Tensor> tensors;
    bool handed_out = false;             // a pointer into the mapping is in use somewhere: never unmap
};

const char* const DTYPES[] = {"F32", "F16", "BF16", "I32", "I64", "U8"};
const int DTYPE_SIZE[] = {4, 2, 2, 4, 8, 1};
constexpr int N_DTYPES = 6;

// ---- a JSON reader, as small as the header needs ---------------------------------------------
struct Json {
    const char* p;
    const char* end;
    std::string err;

    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char* what) { if (err.empty()) err = what; return false; }
    bool expect(char c) {
        ws();
        if (p < end && *p == c) { ++p; return true; }
        return fail("unexpected character");
    }
    bool string(std::string* out) {
        ws();
        if (p >= end || *p != '"') return fail("a string was expected");
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("unfinished escape");
                switch (*p) {
                    case '"': case '\\': case '/': if (out) out->push_back(*p); break;
                    case 'b': if (out) out->push_back('\b'); break;
                    case 'f': if (out) out->push_back('\f'); break;
                    case 'n': if (out) out->push_back('\n'); break;
                    case 'r': if (out) out->push_back('\r'); break;
                    case 't': if (out) out->push_back('\t'); break;
                    case 'u': {
                        if (end - p < 5) return fail("unfinished \\u escape");
                        unsigned cp = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char c = p[i];
                            cp <<= 4;
                            if (c >= '0' && c <= '9') cp |= (unsigned)(c - '0');
                            else if (c >= 'a' && c <= 'f') cp |= (unsigned)(c - 'a' + 10);
                            else if (c >= 'A' && c <= 'F') cp |= (unsigned)(c - 'A' + 10);
                            else return fail("bad \\u escape");
                        }
                        p += 4;
                        if (out) {                          // UTF-8 (surrogate pairs are kept as they come)
                            if (cp < 0x80) out->push_back((char)cp);
                            else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                            else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                        }
                        break;
                    }
                    default: return fail("unknown escape");
                }
                ++p;
            } else {
                if (out) out->push_back(*p);
                ++p;
            }
        }
        if (p >= end) return fail("unfinished string");
        ++p;
        return true;
    }
    bool integer(long long* out) {
        ws();
        const char* s = p;
        bool neg = false;
        if (p < end && *p == '-') { neg = true; ++p; }
        if (p >= end || *p < '0' || *p > '9') { p = s; return fail("an integer was expected"); }
        long long v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (v > (INT64_MAX - 9) / 10) return fail("integer too large");
            v = v * 10 + (*p - '0');
            ++p;
        }
        if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail("an integer was expected, not a fraction");
        *out = neg ? -v : v;
        return true;
    }
    bool int_array(std::vector<long long>* out) {
        if (!expect('[')) return false;
        ws();
        if (p < end && *p == ']') { ++p; return true; }
        for (;;) {
            long long v;
            if (!integer(&v)) return false;
            out->push_back(v);
            ws();
            if (p < end && *p == ',') { ++p; continue; }
            return expect(']');
        }
    }
    bool skip_value() {                                  // any JSON value, contents ignored
        ws();
        if (p >= end) return fail("a value was expected");
        if (*p == '"') return string(nullptr);
        if (*p == '{') {
            ++p; ws();
            if (p < end && *p == '}') { ++p; return true; }
            for (;;) {
                if (!string(nullptr) || !expect(':') || !skip_value()) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                return expect('}');
            }
        }
        if (*p == '[') {
            ++p; ws();
            if (p < end && *p == ']') { ++p; return true; }
            for (;;) {
                if (!skip_value()) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                return expect(']');
            }
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') ++p;
        return true;                                     // number, true, false, null
    }
};

void parse(File& f) {
    char buf[512];
    auto fail = [&](const std::string& msg) { f.error = f.path + ": " + msg; };
    if (f.size < 8) return fail("too short to hold a safetensors header");
    const uint8_t* base = static_cast<const uint8_t*>(f.map);
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | base[i];
    if (hlen == 0 || hlen > f.size - 8) {
        snprintf(buf, sizeof buf, "header length %llu does not fit the file (%zu bytes)", (unsigned long long)hlen, f.size);
        return fail(buf);
    }
    const long long payload = (long long)(f.size - 8 - hlen);
    Json j{reinterpret_cast<const char*>(base + 8), reinterpret_cast<const char*>(base + 8 + hlen), ""};
    auto bad_json = [&]() { fail("header is not valid JSON: " + (j.err.empty() ? std::string("malformed") : j.err)); };
    if (!j.expect('{')) return bad_json();
    j.ws();
    if (j.p < j.end && *j.p == '}') return;              // no tensors
    for (;;) {
        Tensor t;
        if (!j.string(&t.name) || !j.expect(':')) return bad_json();
        if (t.name == "__metadata__") {
            if (!j.skip_value()) return bad_json();
        } else {
            std::string dtype;
            std::vector<long long> offsets;
            bool have_dtype = false, have_shape = false, have_offsets = false;
            if (!j.expect('{')) return bad_json();
            for (;;) {
                std::string key;
                if (!j.string(&key) || !j.expect(':')) return bad_json();
                if (key == "dtype") { if (!j.string(&dtype)) return bad_json(); have_dtype = true; }
                else if (key == "shape") { if (!j.int_array(&t.shape)) return bad_json(); have_shape = true; }
                else if (key == "data_offsets") { if (!j.int_array(&offsets)) return bad_json(); have_offsets = true; }
                else if (!j.skip_value()) return bad_json();
                j.ws();
                if (j.p < j.end && *j.p == ',') { ++j.p; continue; }
                if (!j.expect('}')) return bad_json();
                break;
            }
            if (!have_dtype || !have_shape || !have_offsets || offsets.size() != 2)
                return fail("tensor '" + t.name + "' lacks dtype, shape or data_offsets");
            t.dtype = -1;
            for (int i = 0; i < N_DTYPES; ++i)
                if (dtype == DTYPES[i]) t.dtype = i;
            if (t.dtype < 0) return fail("tensor '" + t.name + "' has unsupported dtype '" + dtype + "'");
            long long n = 1;
            for (long long s : t.shape) {
                if (s < 0 || (s > 0 && n > INT64_MAX / 16 / s)) return fail("tensor '" + t.name + "' has an impossible shape");
                n *= s;
            }
            const long long b = offsets[0], e = offsets[1];
            if (b < 0 || e < b || e > payload) {
                snprintf(buf, sizeof buf, "offsets [%lld, %lld) lie outside the payload", b, e);
                return fail("tensor '" + t.name + "' " + buf);
            }
            if (e - b != n * DTYPE_SIZE[t.dtype]) {
                snprintf(buf, sizeof buf, "holds %lld bytes but its shape of %s needs %lld", e - b, DTYPES[t.dtype],
                         n * DTYPE_SIZE[t.dtype]);
                return fail("tensor '" + t.name + "' " + buf);
            }
            t.begin = 8 + (long long)hlen + b;
            t.nbytes = e - b;
            f.tensors.push_back(std::move(t));
        }
        j.ws();
        if (j.p < j.end && *j.p == ',') { ++j.p; continue; }
        if (!j.expect('}')) return bad_json();
        break;
    }
}

}  // namespace

extern "C" {

// Always returns a handle (null only when out of memory); infero_st_error says whether it is usable.
void* infero_st_open(const char* path) {
    File* f = new File();
    f->path = path;
    f->fd = open(path, O_RDONLY);
    if (f->fd < 0) { f->error = f->path + ": cannot be opened"; return f; }
    struct stat st;
    if (fstat(f->fd, &st) != 0) { f->error = f->path + ": cannot be examined"; return f; }
    f->size = (size_t)st.st_size;
    if (f->size < 8) { f->error = f->path + ": too short to hold a safetensors header"; return f; }
    f->map = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (f->map == MAP_FAILED) { f->map = nullptr; f->error = f->path + ": cannot be mapped"; return f; }
    parse(*f);
    return f;
}

const char* infero_st_error(void* h) { return static_cast<File*>(h)->error.c_str(); }
int infero_st_count(void* h) { return (int)static_cast<File*>(h)->tensors.size(); }
const char* infero_st_name(void* h, int i) { return static_cast<File*>(h)->tensors[i].name.c_str(); }
int infero_st_dtype(void* h, int i) { return static_cast<File*>(h)->tensors[i].dtype; }
int infero_st_rank(void* h, int i) { return (int)static_cast<File*>(h)->tensors[i].shape.size(); }
void infero_st_shape(void* h, int i, long long* out) {
    const Tensor& t = static_cast<File*>(h)->tensors[i];
    for (size_t k = 0; k < t.shape.size(); ++k) out[k] = t.shape[k];
}
long long infero_st_nbytes(void* h, int i) { return static_cast<File*>(h)->tensors[i].nbytes; }
long long infero_st_offset(void* h, int i) { return static_cast<File*>(h)->tensors[i].begin; }
// The tensor's bytes inside the mapping; the mapping then stays for the life of the process.
const void* infero_st_data(void* h, int i) {
    File* f = static_cast<File*>(h);
    f->handed_out = true;
    return static_cast<const uint8_t*>(f->map) + f->tensors[i].begin;
}

void infero_st_close(void* h) {
    File* f = static_cast<File*>(h);
    if (f->map && !f->handed_out) munmap(f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    if (!f->handed_out) delete f;                        // (else the names and the mapping stay, like the pointers)
    else f->fd = -1;
}

}  // extern "C"
