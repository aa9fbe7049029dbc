// Checkpoint files in the reference's two formats (src/engine/model/checkpoint.rs), so that a
// checkpoint written here loads in Volta and the other way round.  Host code only.
#include "vb_checkpoint.h"

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace vb {

namespace {

const char kHeaderPrefix[] = "#volta-checkpoint:";
const char kMagic[8] = {'V', 'O', 'L', 'T', 'A', 2, 0, 0};

bool fail(std::string *err, const std::string &msg) {
    if (err) *err = msg;
    return false;
}

std::string trim(const std::string &s) {
    size_t a = 0, b = s.size();
    while (a < b && (s[a] == ' ' || s[a] == '\t' || s[a] == '\r' || s[a] == '\n')) ++a;
    while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\t' || s[b - 1] == '\r' || s[b - 1] == '\n')) --b;
    return s.substr(a, b - a);
}

bool product_matches(const std::vector<int64_t> &shape, size_t count) {
    unsigned long long p = 1;
    for (int64_t d : shape) {
        if (d < 0) return false;
        p *= (unsigned long long)d;
        if (p > (1ULL << 40)) return false;
    }
    return p == count;
}

bool read_file(const std::string &path, std::string *out, std::string *err) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return fail(err, "Failed to read checkpoint from '" + path + "': " + strerror(errno));
    char buf[1 << 16];
    size_t n;
    out->clear();
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out->append(buf, n);
    fclose(f);
    return true;
}

bool write_file(const std::string &path, const std::string &bytes, std::string *err) {
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) return fail(err, "Failed to save checkpoint to '" + path + "': " + strerror(errno));
    const bool ok = fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size();
    if (fclose(f) != 0 || !ok) return fail(err, "Failed to save checkpoint to '" + path + "': short write");
    return true;
}

std::vector<const CheckpointEntry *> sorted(const Checkpoint &ck) {
    std::vector<const CheckpointEntry *> v;
    for (auto &e : ck.entries) v.push_back(&e);
    std::sort(v.begin(), v.end(), [](const CheckpointEntry *a, const CheckpointEntry *b) { return a->name < b->name; });
    return v;
}

// ---- v1 text ---------------------------------------------------------------------------------
// One value as the reference writes it, `{v:.9}` (checkpoint.rs:35): fixed notation, nine decimals.
// That form loses small magnitudes (1.2345678e-7 becomes 0.000000123); the default writer therefore
// prints nine SIGNIFICANT digits, which every fp32 value survives bit for bit and which the
// reference's reader parses the same way.
void print_value(char *buf, size_t cap, float v, bool fixed9) {
    if (v != v) { snprintf(buf, cap, "NaN"); return; }                        // Rust prints NaN, C prints nan
    if (fixed9 && (v - v) != 0.0f) { snprintf(buf, cap, v < 0 ? "-inf" : "inf"); return; }
    snprintf(buf, cap, fixed9 ? "%.9f" : "%.9g", (double)v);
}

std::string to_text(const Checkpoint &ck, bool fixed9) {
    std::string out = std::string(kHeaderPrefix) + "v1\n#writer:volta_b200";
    char num[64];
    for (const CheckpointEntry *e : sorted(ck)) {
        out += "\n" + e->name + "|";
        for (size_t i = 0; i < e->shape.size(); ++i) {
            snprintf(num, sizeof num, "%s%lld", i ? "," : "", (long long)e->shape[i]);
            out += num;
        }
        out += "|";
        for (size_t i = 0; i < e->data.size(); ++i) {
            if (i) out += ",";
            print_value(num, sizeof num, e->data[i], fixed9);
            out += num;
        }
    }
    return out;
}

// true: the line is a version header (and the version is one this reader knows)
bool header_line(const std::string &line, size_t line_no, bool *is_header, std::string *err) {
    const std::string t = trim(line);
    *is_header = t.compare(0, sizeof(kHeaderPrefix) - 1, kHeaderPrefix) == 0;
    if (!*is_header) return true;
    const std::string version = t.substr(sizeof(kHeaderPrefix) - 1);
    if (version != "v1")
        return fail(err, "Unsupported checkpoint version '" + version + "' at line " + std::to_string(line_no + 1));
    return true;
}

// The grammar of Rust's f32::from_str, which the reference's reader applies to every value
// (checkpoint.rs:141): optional sign, then inf / infinity / nan in any case, or decimal digits with
// an optional point and an optional decimal exponent.  No whitespace, no hexadecimal floats, no
// digit separators; strtof alone would accept the first two.
bool is_rust_f32(const std::string &t) {
    size_t i = 0;
    if (i < t.size() && (t[i] == '+' || t[i] == '-')) ++i;
    std::string rest = t.substr(i);
    for (char &c : rest) c = (char)tolower((unsigned char)c);
    if (rest == "inf" || rest == "infinity" || rest == "nan") return true;
    size_t digits = 0;
    while (i < t.size() && isdigit((unsigned char)t[i])) { ++i; ++digits; }
    if (i < t.size() && t[i] == '.') {
        ++i;
        while (i < t.size() && isdigit((unsigned char)t[i])) { ++i; ++digits; }
    }
    if (digits == 0) return false;
    if (i < t.size() && (t[i] == 'e' || t[i] == 'E')) {
        ++i;
        if (i < t.size() && (t[i] == '+' || t[i] == '-')) ++i;
        size_t ed = 0;
        while (i < t.size() && isdigit((unsigned char)t[i])) { ++i; ++ed; }
        if (ed == 0) return false;
    }
    return i == t.size();
}

bool parse_entry(const std::string &line, size_t line_no, CheckpointEntry *e, std::string *err) {
    const std::string at = " at line " + std::to_string(line_no + 1);
    const size_t p1 = line.find('|');
    const size_t p2 = p1 == std::string::npos ? p1 : line.find('|', p1 + 1);
    if (p2 == std::string::npos || line.find('|', p2 + 1) != std::string::npos)
        return fail(err, "Invalid checkpoint format" + at);
    e->name = line.substr(0, p1);
    e->shape.clear();
    e->data.clear();
    const std::string shape = line.substr(p1 + 1, p2 - p1 - 1), data = line.substr(p2 + 1);
    for (size_t p = 0; !shape.empty() && p <= shape.size();) {
        size_t q = shape.find(',', p);
        if (q == std::string::npos) q = shape.size();
        const std::string tok = shape.substr(p, q - p);
        char *end = nullptr;
        errno = 0;
        unsigned long long v = strtoull(tok.c_str(), &end, 10);
        if (tok.empty() || *end || errno || tok[0] == '-' || tok[0] == '+' || tok[0] == ' ')
            return fail(err, "Invalid shape dimension '" + tok + "'" + at);
        e->shape.push_back((int64_t)v);
        p = q + 1;
    }
    for (size_t p = 0; !data.empty() && p <= data.size();) {
        size_t q = data.find(',', p);
        if (q == std::string::npos) q = data.size();
        const std::string tok = data.substr(p, q - p);
        char *end = nullptr;
        float v = strtof(tok.c_str(), &end);
        if (!is_rust_f32(tok) || *end) return fail(err, "Invalid data value '" + tok + "'" + at);
        e->data.push_back(v);
        p = q + 1;
    }
    if (!product_matches(e->shape, e->data.size()))
        return fail(err, "Invalid tensor in checkpoint" + at + ": shape does not match the number of values");
    return true;
}

bool from_text(const std::string &text, Checkpoint *ck, std::string *err) {
    size_t line_no = 0;
    for (size_t p = 0; p <= text.size(); ++line_no) {
        size_t q = text.find('\n', p);
        if (q == std::string::npos) q = text.size();
        const std::string line = text.substr(p, q - p);
        p = q + 1;
        const std::string t = trim(line);
        if (t.empty()) continue;
        bool is_header = false;
        if (!header_line(line, line_no, &is_header, err)) return false;
        if (is_header || t[0] == '#') continue;
        CheckpointEntry e;
        if (!parse_entry(t, line_no, &e, err)) return false;
        ck->put(e.name, e.shape, e.data.data(), e.data.size());
    }
    return true;
}

// ---- v2 binary -------------------------------------------------------------------------------
void put_u16(std::string &s, uint16_t v) { s.push_back((char)(v & 255)); s.push_back((char)(v >> 8)); }
void put_u32(std::string &s, uint32_t v) { for (int i = 0; i < 4; ++i) s.push_back((char)((v >> (8 * i)) & 255)); }

uint32_t adler32(const std::string &d) {
    uint32_t a = 1, b = 0;
    for (unsigned char c : d) {
        a = (a + c) % 65521u;
        b = (b + a) % 65521u;
    }
    return (b << 16) | a;
}

// zlib framing around stored deflate blocks of at most 65535 bytes (checkpoint.rs:293-320)
std::string zlib_stored(const std::string &payload) {
    std::string out;
    out.push_back((char)0x78);
    out.push_back((char)0x9C);
    size_t p = 0;
    while (p < payload.size()) {
        const size_t len = std::min<size_t>(65535, payload.size() - p);
        const bool last = p + len == payload.size();
        out.push_back(last ? 1 : 0);
        put_u16(out, (uint16_t)len);
        put_u16(out, (uint16_t)~(uint16_t)len);
        out.append(payload, p, len);
        p += len;
    }
    const uint32_t ad = adler32(payload);
    for (int i = 3; i >= 0; --i) out.push_back((char)((ad >> (8 * i)) & 255));
    return out;
}

bool unzlib_stored(const std::string &z, std::string *out, std::string *err) {
    if (z.size() < 6) return fail(err, "Compressed data too short");
    size_t pos = 2;
    out->clear();
    for (;;) {
        if (pos >= z.size()) return fail(err, "Unexpected end in deflate stream");
        const unsigned char hdr = (unsigned char)z[pos++];
        const int btype = (hdr >> 1) & 3;
        if (btype != 0)
            return fail(err, "Compressed deflate BTYPE=" + std::to_string(btype) + " not supported in this decompressor");
        if (pos + 4 > z.size()) return fail(err, "Truncated deflate block header");
        const size_t len = (unsigned char)z[pos] | ((size_t)(unsigned char)z[pos + 1] << 8);
        pos += 4;
        if (pos + len > z.size()) return fail(err, "Truncated deflate block data");
        out->append(z, pos, len);
        pos += len;
        if (hdr & 1) break;
    }
    return true;
}

struct Reader {
    const std::string &b;
    size_t pos = 0;
    bool ok = true;
    bool need(size_t n) {
        if (pos + n > b.size()) ok = false;
        return ok;
    }
    uint32_t u32() {
        if (!need(4)) return 0;
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) v |= (uint32_t)(unsigned char)b[pos + i] << (8 * i);
        pos += 4;
        return v;
    }
    uint16_t u16() {
        if (!need(2)) return 0;
        uint16_t v = (uint16_t)((unsigned char)b[pos] | ((unsigned char)b[pos + 1] << 8));
        pos += 2;
        return v;
    }
};

std::string to_binary(const Checkpoint &ck, std::string *err) {
    std::string payload;
    put_u32(payload, (uint32_t)ck.entries.size());
    for (const CheckpointEntry *e : sorted(ck)) {
        if (e->name.size() > 65535 || e->data.size() > 0xffffffffULL) {
            fail(err, "entry '" + e->name + "' does not fit the binary format");
            return std::string();
        }
        put_u16(payload, (uint16_t)e->name.size());
        payload += e->name;
        put_u32(payload, (uint32_t)e->shape.size());
        for (int64_t d : e->shape) put_u32(payload, (uint32_t)d);
        put_u32(payload, (uint32_t)e->data.size());
        const size_t at = payload.size();
        payload.resize(at + e->data.size() * 4);
        for (size_t i = 0; i < e->data.size(); ++i) {
            uint32_t bits;
            memcpy(&bits, &e->data[i], 4);
            for (int k = 0; k < 4; ++k) payload[at + 4 * i + k] = (char)((bits >> (8 * k)) & 255);
        }
    }
    return std::string(kMagic, 8) + zlib_stored(payload);
}

bool from_binary(const std::string &z, Checkpoint *ck, std::string *err) {
    std::string payload;
    if (!unzlib_stored(z, &payload, err)) return false;
    Reader r{payload};
    const uint32_t count = r.u32();
    for (uint32_t i = 0; i < count && r.ok; ++i) {
        CheckpointEntry e;
        const uint16_t nl = r.u16();
        if (!r.need(nl)) break;
        e.name.assign(payload, r.pos, nl);
        r.pos += nl;
        const uint32_t ndim = r.u32();
        if (!r.need((size_t)ndim * 4)) break;
        for (uint32_t d = 0; d < ndim; ++d) e.shape.push_back(r.u32());
        const uint32_t ne = r.u32();
        if (!r.need((size_t)ne * 4)) break;
        e.data.resize(ne);
        for (uint32_t k = 0; k < ne; ++k) {
            uint32_t bits = r.u32();
            memcpy(&e.data[k], &bits, 4);
        }
        if (!product_matches(e.shape, e.data.size()))
            return fail(err, "Invalid tensor for '" + e.name + "': shape does not match the number of values");
        ck->put(e.name, e.shape, e.data.data(), e.data.size());
    }
    if (!r.ok) return fail(err, "Unexpected end of checkpoint data");
    return true;
}

}  // namespace

const CheckpointEntry *Checkpoint::find(const std::string &name) const {
    for (auto &e : entries)
        if (e.name == name) return &e;
    return nullptr;
}

void Checkpoint::put(const std::string &name, const std::vector<int64_t> &shape, const float *data, size_t count) {
    CheckpointEntry *dst = nullptr;
    for (auto &e : entries)
        if (e.name == name) dst = &e;
    if (!dst) {
        entries.emplace_back();
        dst = &entries.back();
        dst->name = name;
    }
    dst->shape = shape;
    dst->data.assign(data, data + count);
}

bool checkpoint_save(const Checkpoint &ck, const std::string &path, int format, std::string *err) {
    for (auto &e : ck.entries) {
        if (e.name.empty() || e.name.find_first_of("|\n\r") != std::string::npos || e.name[0] == '#')
            return fail(err, "entry name '" + e.name + "' cannot be written");
        if (!product_matches(e.shape, e.data.size())) return fail(err, "entry '" + e.name + "': shape does not match its data");
    }
    if (format == 1) return write_file(path, to_text(ck, false), err);
    if (format == 3) return write_file(path, to_text(ck, true), err);
    if (format == 2) {
        std::string e2;
        std::string bytes = to_binary(ck, &e2);
        if (bytes.empty()) return fail(err, e2);
        return write_file(path, bytes, err);
    }
    return fail(err, "unknown checkpoint format (1 = v1 text, 2 = v2 binary, 3 = v1 text with the reference's nine fixed decimals)");
}

bool checkpoint_parse(Checkpoint *ck, const std::string &raw, std::string *err) {
    ck->entries.clear();
    if (raw.size() >= 8 && memcmp(raw.data(), kMagic, 8) == 0) return from_binary(raw.substr(8), ck, err);
    return from_text(raw, ck, err);
}

bool checkpoint_load(Checkpoint *ck, const std::string &path, std::string *err) {
    std::string raw;
    if (!read_file(path, &raw, err)) return false;
    return checkpoint_parse(ck, raw, err);
}

void split_u64(uint64_t v, float out[3]) {
    out[0] = (float)(v & 0x3fffffULL);
    out[1] = (float)((v >> 22) & 0x3fffffULL);
    out[2] = (float)(v >> 44);
}

bool join_u64(const float in[3], uint64_t *v) {
    uint64_t parts[3];
    for (int i = 0; i < 3; ++i) {
        if (!(in[i] >= 0.0f) || in[i] > 4194303.0f || in[i] != (float)(uint64_t)in[i]) return false;
        parts[i] = (uint64_t)in[i];
    }
    if (parts[2] > 0xfffffULL) return false;
    *v = parts[0] | (parts[1] << 22) | (parts[2] << 44);
    return true;
}

}  // namespace vb
