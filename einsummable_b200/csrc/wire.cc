// Interchange formats of the callers either side of the hot path.
//
// (1) The protobuf messages of src/proto/einsummable.proto (proto2) that carry graphs between
//     processes -- memgraph_t::to_wire / from_wire (src/einsummable/memgraph.cc:258-380, used when a
//     server broadcasts the memgraph to its workers, src/server/mg_base.cc:118), taskgraph_t,
//     einsummable_t, touch_t, fill_t, partitions and placements -- as a schema-driven codec between
//     the protobuf wire format and JSON with the .proto's field names.  No protobuf library and no
//     generated code: the wire format is varints and length-delimited fields, and proto2 writes
//     repeated scalars one tag per element (packed input is accepted as well).
// (2) The weight file the reference's converter writes and its reader reads (llama/from_pth2.py:27-35,
//     llama/reader.cc:42-110): records of a 50-byte space-padded name, an int64 element count and
//     that many f16 values.
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.h"

namespace {

using namespace es;

enum ftype_t { T_INT32, T_INT64, T_UINT64, T_BOOL, T_STRING, T_MESSAGE };

struct field_t {
    int         number;
    char const* name;
    ftype_t     type;
    bool        repeated;
    char const* message; // T_MESSAGE: the field's message type
};

using schema_t = std::map<std::string, std::vector<field_t>>;

#define S(n, name, type) {n, name, type, false, nullptr}
#define R(n, name, type) {n, name, type, true, nullptr}
#define M(n, name, msg) {n, name, T_MESSAGE, false, msg}
#define RM(n, name, msg) {n, name, T_MESSAGE, true, msg}

schema_t const& schema()
{
    static schema_t const s = {
        {"EsInn", {R(1, "idxs", T_INT32)}},
        {"Einsummable", {R(1, "join_shape", T_UINT64), RM(2, "inns", "EsInn"), S(3, "out_rank", T_INT32),
                         S(4, "join", T_STRING), S(5, "castable", T_STRING)}},
        {"EinsummableList", {RM(1, "es", "Einsummable")}},
        {"TouchDim", {S(1, "d_inn", T_UINT64), S(2, "d_out", T_UINT64), S(3, "offset_inn", T_UINT64),
                      S(4, "offset_out", T_UINT64), S(5, "size", T_UINT64)}},
        {"Touch", {RM(1, "selection", "TouchDim"), S(2, "castable", T_STRING), S(3, "dtype", T_STRING)}},
        {"Constant", {S(1, "value", T_STRING), R(2, "shape", T_UINT64)}},
        {"Lowertri", {S(1, "lower", T_STRING), S(2, "upper", T_STRING), S(3, "ncol", T_UINT64),
                      S(4, "nrow", T_UINT64), S(5, "start", T_INT64)}},
        {"Fill", {M(1, "constant", "Constant"), M(2, "lowertri", "Lowertri")}},
        {"TGInput", {S(1, "loc", T_INT32), S(2, "size", T_UINT64)}},
        {"TGApply", {S(1, "loc", T_INT32), R(2, "inns", T_INT32), M(3, "einsummable", "Einsummable")}},
        {"TGMove", {S(1, "src", T_INT32), S(2, "dst", T_INT32), S(3, "inn", T_INT32), S(4, "size", T_UINT64)}},
        {"TGConstant", {S(1, "loc", T_INT32), M(2, "fill", "Fill")}},
        {"InnRegionDim", {S(1, "dim", T_UINT64), S(2, "offset", T_UINT64)}},
        {"OutRegionDim", {S(1, "offset", T_UINT64), S(2, "size", T_UINT64)}},
        {"TGPartialInn", {S(1, "id", T_INT32), S(2, "consumable", T_BOOL), RM(3, "region", "InnRegionDim")}},
        {"TGPartialUnit", {S(1, "castable", T_STRING), RM(2, "out_region", "OutRegionDim"),
                           RM(3, "inputs", "TGPartialInn")}},
        {"TGPartialize", {S(1, "loc", T_INT32), S(2, "dtype", T_STRING), R(3, "write_shape", T_UINT64),
                          RM(4, "units", "TGPartialUnit")}},
        {"TaskGraphNode", {M(1, "input", "TGInput"), M(2, "apply", "TGApply"), M(3, "move", "TGMove"),
                           M(4, "constant", "TGConstant"), M(5, "partialize", "TGPartialize"),
                           S(6, "is_save", T_BOOL)}},
        {"TaskGraph", {RM(1, "nodes", "TaskGraphNode")}},
        {"Partdim", {R(1, "spans", T_UINT64)}},
        {"Partition", {RM(1, "partdims", "Partdim")}},
        {"Placement", {M(1, "partition", "Partition"), R(2, "locations", T_INT32)}},
        {"Relation", {S(1, "dtype", T_STRING), M(2, "placement", "Placement"), R(4, "tids", T_INT32)}},
        {"RemapRelations", {RM(1, "srcs", "Relation"), RM(2, "dsts", "Relation")}},
        {"MGInputMem", {S(1, "loc", T_INT32), S(2, "offset", T_UINT64), S(3, "size", T_UINT64)}},
        {"MGInputSto", {S(1, "storage_loc", T_INT32), S(2, "storage_id", T_INT32), S(3, "size", T_UINT64)}},
        {"MGConstant", {S(1, "loc", T_INT32), S(2, "offset", T_UINT64), M(3, "fill", "Fill")}},
        {"MGApply", {S(1, "loc", T_INT32), R(2, "mems_offset", T_UINT64), R(3, "mems_size", T_UINT64),
                     M(4, "einsummable", "Einsummable"), M(5, "touch", "Touch"), S(6, "group", T_INT32)}},
        {"MGMove", {S(1, "src_loc", T_INT32), S(2, "src_offset", T_UINT64), S(3, "dst_loc", T_INT32),
                    S(4, "dst_offset", T_UINT64), S(5, "size", T_UINT64)}},
        {"MGCopy", {S(1, "loc", T_INT32), S(2, "size", T_UINT64), S(3, "src_offset", T_UINT64),
                    S(4, "dst_offset", T_UINT64)}},
        {"MGEvict", {S(1, "storage_loc", T_INT32), S(2, "storage_id", T_INT32), S(3, "loc", T_INT32),
                     S(4, "offset", T_UINT64), S(5, "size", T_UINT64)}},
        {"MGLoad", {S(1, "storage_loc", T_INT32), S(2, "storage_id", T_INT32), S(3, "loc", T_INT32),
                    S(4, "offset", T_UINT64), S(5, "size", T_UINT64)}},
        {"MGPartialize", {S(1, "loc", T_INT32), S(2, "offset", T_UINT64), S(3, "size", T_UINT64)}},
        {"MGAlloc", {S(1, "loc", T_INT32), S(2, "offset", T_UINT64), S(3, "size", T_UINT64)}},
        {"MGDel", {S(1, "loc", T_INT32), S(2, "offset", T_UINT64), S(3, "size", T_UINT64)}},
        {"MemGraphNode", {M(1, "inputmem", "MGInputMem"), M(2, "inputsto", "MGInputSto"),
                          M(3, "constant", "MGConstant"), M(4, "apply", "MGApply"), M(5, "move", "MGMove"),
                          M(6, "evict", "MGEvict"), M(7, "load", "MGLoad"), M(8, "partialize", "MGPartialize"),
                          M(9, "alloc", "MGAlloc"), M(10, "del", "MGDel"), R(11, "inns", T_INT32),
                          M(100, "copy", "MGCopy")}},
        {"MemGraph", {S(1, "num_compute_locs", T_INT32), S(2, "num_storage_locs", T_INT32),
                      R(3, "storage_locs", T_INT32), RM(4, "nodes", "MemGraphNode")}},
        {"Mem", {S(1, "offset", T_UINT64), S(2, "size", T_UINT64)}},
        {"MemLoc", {S(1, "offset", T_UINT64), S(2, "size", T_UINT64), S(3, "loc", T_INT32)}},
    };
    return s;
}

std::vector<field_t> const& fields_of(std::string const& msg)
{
    auto it = schema().find(msg);
    if (it == schema().end()) fail(ES_BAD_ARGUMENT, "wire: unknown message type " + msg);
    return it->second;
}

// ---------------------------------------------------------------- wire -> JSON
struct reader_t {
    unsigned char const* p;
    unsigned char const* end;
    uint64_t varint()
    {
        uint64_t v = 0;
        for (int shift = 0; shift < 70; shift += 7) {
            if (p == end) fail(ES_BAD_DESCRIPTOR, "wire: truncated varint");
            unsigned char b = *p++;
            v |= (uint64_t)(b & 0x7f) << shift;
            if (!(b & 0x80)) return v;
        }
        fail(ES_BAD_DESCRIPTOR, "wire: varint too long");
    }
};

void json_string(std::string& out, char const* s, size_t n)
{
    out += '"';
    for (size_t i = 0; i != n; ++i) {
        unsigned char c = (unsigned char)s[i];
        if (c == '"' || c == '\\') {
            out += '\\';
            out += (char)c;
        } else if (c < 0x20) {
            char buf[8];
            std::snprintf(buf, sizeof buf, "\\u%04x", c);
            out += buf;
        } else {
            out += (char)c;
        }
    }
    out += '"';
}

void scalar_json(std::string& out, ftype_t t, uint64_t v)
{
    if (t == T_BOOL) out += v ? "true" : "false";
    else if (t == T_UINT64) out += std::to_string(v);
    else if (t == T_INT32) out += std::to_string((int32_t)(int64_t)v);
    else out += std::to_string((int64_t)v);
}

std::string decode(std::string const& msg, unsigned char const* data, size_t n, int depth)
{
    if (depth > 32) fail(ES_BAD_DESCRIPTOR, "wire: nesting too deep");
    auto const&                              fields = fields_of(msg);
    std::map<int, std::vector<std::string>>  values; // field number -> rendered values
    reader_t                                 r{data, data + n};
    while (r.p != r.end) {
        uint64_t tag = r.varint();
        int      number = (int)(tag >> 3), wt = (int)(tag & 7);
        field_t const* f = nullptr;
        for (auto const& x : fields)
            if (x.number == number) f = &x;
        if (wt == 0) {
            uint64_t v = r.varint();
            if (f && f->type != T_STRING && f->type != T_MESSAGE) {
                std::string s;
                scalar_json(s, f->type, v);
                values[number].push_back(s);
            }
        } else if (wt == 2) {
            uint64_t len = r.varint();
            if (len > (uint64_t)(r.end - r.p)) fail(ES_BAD_DESCRIPTOR, "wire: truncated field");
            if (f && f->type == T_STRING) {
                std::string s;
                json_string(s, (char const*)r.p, len);
                values[number].push_back(s);
            } else if (f && f->type == T_MESSAGE) {
                values[number].push_back(decode(f->message, r.p, len, depth + 1));
            } else if (f) { // packed repeated scalars
                reader_t q{r.p, r.p + len};
                while (q.p != q.end) {
                    std::string s;
                    scalar_json(s, f->type, q.varint());
                    values[number].push_back(s);
                }
            }
            r.p += len;
        } else if (wt == 1) {
            if (r.end - r.p < 8) fail(ES_BAD_DESCRIPTOR, "wire: truncated fixed64");
            r.p += 8;
        } else if (wt == 5) {
            if (r.end - r.p < 4) fail(ES_BAD_DESCRIPTOR, "wire: truncated fixed32");
            r.p += 4;
        } else {
            fail(ES_BAD_DESCRIPTOR, "wire: unsupported wire type " + std::to_string(wt));
        }
    }
    std::string out = "{";
    bool        first = true;
    for (auto const& f : fields) {
        auto it = values.find(f.number);
        if (it == values.end() && !f.repeated) continue;
        out += first ? "" : ", ";
        first = false;
        json_string(out, f.name, std::strlen(f.name));
        out += ": ";
        if (f.repeated) {
            out += "[";
            if (it != values.end())
                for (size_t i = 0; i != it->second.size(); ++i) out += (i ? ", " : "") + it->second[i];
            out += "]";
        } else {
            out += it->second.back(); // the last occurrence wins
        }
    }
    return out + "}";
}

// ---------------------------------------------------------------- JSON -> wire
struct jvalue_t {
    enum { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool                                          b = false;
    std::string                                   text; // number text or string
    std::vector<jvalue_t>                         arr;
    std::vector<std::pair<std::string, jvalue_t>> obj;
};

struct jparser_t {
    char const* p;
    void        ws()
    {
        while (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r') ++p;
    }
    jvalue_t value(int depth)
    {
        if (depth > 64) fail(ES_BAD_DESCRIPTOR, "json: nesting too deep");
        ws();
        jvalue_t v;
        if (*p == '{') {
            v.kind = jvalue_t::OBJ;
            ++p;
            ws();
            if (*p == '}') {
                ++p;
                return v;
            }
            while (true) {
                ws();
                jvalue_t k = value(depth + 1);
                if (k.kind != jvalue_t::STR) fail(ES_BAD_DESCRIPTOR, "json: object key must be a string");
                ws();
                if (*p++ != ':') fail(ES_BAD_DESCRIPTOR, "json: expected ':'");
                v.obj.emplace_back(k.text, value(depth + 1));
                ws();
                if (*p == ',') {
                    ++p;
                    continue;
                }
                if (*p++ != '}') fail(ES_BAD_DESCRIPTOR, "json: expected '}'");
                return v;
            }
        }
        if (*p == '[') {
            v.kind = jvalue_t::ARR;
            ++p;
            ws();
            if (*p == ']') {
                ++p;
                return v;
            }
            while (true) {
                v.arr.push_back(value(depth + 1));
                ws();
                if (*p == ',') {
                    ++p;
                    continue;
                }
                if (*p++ != ']') fail(ES_BAD_DESCRIPTOR, "json: expected ']'");
                return v;
            }
        }
        if (*p == '"') {
            v.kind = jvalue_t::STR;
            ++p;
            while (*p && *p != '"') {
                if (*p == '\\') {
                    ++p;
                    if (*p == 'n') v.text += '\n';
                    else if (*p == 't') v.text += '\t';
                    else if (*p == 'u') {
                        unsigned code = 0;
                        for (int i = 0; i != 4; ++i) {
                            ++p;
                            code = code * 16 + (unsigned)(*p <= '9' ? *p - '0' : (*p | 32) - 'a' + 10);
                        }
                        v.text += (char)code;
                    } else v.text += *p;
                    ++p;
                } else {
                    v.text += *p++;
                }
            }
            if (*p++ != '"') fail(ES_BAD_DESCRIPTOR, "json: unterminated string");
            return v;
        }
        if (!std::strncmp(p, "true", 4)) {
            p += 4;
            v.kind = jvalue_t::BOOL;
            v.b = true;
            return v;
        }
        if (!std::strncmp(p, "false", 5)) {
            p += 5;
            v.kind = jvalue_t::BOOL;
            return v;
        }
        if (!std::strncmp(p, "null", 4)) {
            p += 4;
            return v;
        }
        v.kind = jvalue_t::NUM;
        while (*p == '-' || *p == '+' || (*p >= '0' && *p <= '9')) v.text += *p++;
        if (v.text.empty()) fail(ES_BAD_DESCRIPTOR, "json: unexpected character");
        return v;
    }
};

void put_varint(std::string& out, uint64_t v)
{
    while (v >= 0x80) {
        out += (char)((v & 0x7f) | 0x80);
        v >>= 7;
    }
    out += (char)v;
}

uint64_t number_of(jvalue_t const& v, ftype_t t)
{
    if (t == T_BOOL) {
        if (v.kind != jvalue_t::BOOL) fail(ES_BAD_DESCRIPTOR, "json: expected a boolean");
        return v.b ? 1 : 0;
    }
    if (v.kind != jvalue_t::NUM) fail(ES_BAD_DESCRIPTOR, "json: expected a number");
    if (t == T_UINT64) return std::stoull(v.text);
    return (uint64_t)(int64_t)std::stoll(v.text); // negative int32 / int64: sign-extended, ten bytes
}

std::string encode(std::string const& msg, jvalue_t const& v, int depth);

void encode_one(std::string& out, field_t const& f, jvalue_t const& v, int depth)
{
    if (f.type == T_STRING) {
        if (v.kind != jvalue_t::STR) fail(ES_BAD_DESCRIPTOR, std::string("json: field ") + f.name + " must be a string");
        put_varint(out, (uint64_t)f.number << 3 | 2);
        put_varint(out, v.text.size());
        out += v.text;
    } else if (f.type == T_MESSAGE) {
        std::string sub = encode(f.message, v, depth + 1);
        put_varint(out, (uint64_t)f.number << 3 | 2);
        put_varint(out, sub.size());
        out += sub;
    } else {
        put_varint(out, (uint64_t)f.number << 3);
        put_varint(out, number_of(v, f.type));
    }
}

std::string encode(std::string const& msg, jvalue_t const& v, int depth)
{
    if (v.kind != jvalue_t::OBJ) fail(ES_BAD_DESCRIPTOR, "json: message " + msg + " must be an object");
    auto const& fields = fields_of(msg);
    for (auto const& kv : v.obj) {
        bool known = false;
        for (auto const& f : fields) known = known || kv.first == f.name;
        if (!known) fail(ES_BAD_DESCRIPTOR, "json: message " + msg + " has no field " + kv.first);
    }
    std::string out;
    // fields in number order, as protobuf serialises them (the table is in number order)
    for (auto const& f : fields) {
        for (auto const& kv : v.obj) {
            if (kv.first != f.name || kv.second.kind == jvalue_t::NUL) continue;
            if (f.repeated) {
                if (kv.second.kind != jvalue_t::ARR) fail(ES_BAD_DESCRIPTOR, std::string("json: field ") + f.name + " must be an array");
                for (auto const& x : kv.second.arr) encode_one(out, f, x, depth);
            } else {
                encode_one(out, f, kv.second, depth);
            }
        }
    }
    return out;
}

template <typename F> int guarded(F&& f)
{
    try {
        f();
        return ES_OK;
    } catch (es_error const& e) {
        set_last_error(e.what());
        return e.status;
    } catch (std::exception const& e) {
        set_last_error(e.what());
        return ES_BAD_ARGUMENT;
    }
}

void give(std::string const& s, void* buf, uint64_t buf_len, uint64_t* needed, bool terminate)
{
    uint64_t n = s.size() + (terminate ? 1 : 0);
    if (needed) *needed = n;
    if (!buf) {
        if (needed) return;
        fail(ES_BAD_ARGUMENT, "wire: null buffer");
    }
    if (buf_len < n) fail(ES_BAD_ARGUMENT, "wire: buffer too small, need " + std::to_string(n));
    std::memcpy(buf, s.data(), s.size());
    if (terminate) static_cast<char*>(buf)[s.size()] = 0;
}

// ---------------------------------------------------------------- weight files
constexpr int NAME_BYTES = 50;

struct file_t {
    std::FILE* f = nullptr;
    file_t(char const* path, char const* mode) : f(std::fopen(path, mode))
    {
        if (!f) fail(ES_BAD_ARGUMENT, std::string("weight file: cannot open ") + path);
    }
    ~file_t()
    {
        if (f) std::fclose(f);
    }
};

bool next_record(std::FILE* f, std::string& name, uint64_t& nelem)
{
    char   raw[NAME_BYTES];
    size_t got = std::fread(raw, 1, NAME_BYTES, f);
    if (got == 0) return false;
    if (got != NAME_BYTES) fail(ES_BAD_DESCRIPTOR, "weight file: truncated record name");
    int64_t count = 0;
    if (std::fread(&count, sizeof count, 1, f) != 1 || count < 0)
        fail(ES_BAD_DESCRIPTOR, "weight file: truncated or negative element count");
    size_t len = NAME_BYTES;
    while (len > 0 && raw[len - 1] == ' ') --len;
    name.assign(raw, len);
    nelem = (uint64_t)count;
    return true;
}

} // namespace

extern "C" {

int es_b200_wire_to_json(const char* message, const void* bytes, uint64_t n, char* buf, uint64_t buf_len,
                         uint64_t* needed)
{
    return guarded([&] {
        if (!message || (!bytes && n)) fail(ES_BAD_ARGUMENT, "wire: null pointer");
        give(decode(message, static_cast<unsigned char const*>(bytes), n, 0), buf, buf_len, needed, true);
    });
}

int es_b200_wire_from_json(const char* message, const char* json, void* buf, uint64_t buf_len, uint64_t* needed)
{
    return guarded([&] {
        if (!message || !json) fail(ES_BAD_ARGUMENT, "wire: null pointer");
        jparser_t parser{json};
        jvalue_t  v = parser.value(0);
        parser.ws();
        if (*parser.p) fail(ES_BAD_DESCRIPTOR, "json: trailing characters");
        give(encode(message, v, 0), buf, buf_len, needed, false);
    });
}

int es_b200_weight_file_list(const char* path, char* names, uint64_t names_len, uint64_t* nelems, int max_records,
                             int* count)
{
    return guarded([&] {
        if (!path || !count) fail(ES_BAD_ARGUMENT, "weight file: null pointer");
        file_t      file(path, "rb");
        std::string all, name;
        uint64_t    nelem = 0;
        int         n = 0;
        while (next_record(file.f, name, nelem)) {
            if (nelems && n < max_records) nelems[n] = nelem;
            all += name;
            all += '\n';
            ++n;
            // every tensor is stored as f16 (llama/reader.cc:22-23)
            if (std::fseek(file.f, (long)(nelem * 2), SEEK_CUR) != 0) fail(ES_BAD_DESCRIPTOR, "weight file: truncated data");
        }
        *count = n;
        if (names) {
            if (names_len < all.size() + 1) fail(ES_BAD_ARGUMENT, "weight file: name buffer too small");
            std::memcpy(names, all.c_str(), all.size() + 1);
        }
    });
}

int es_b200_weight_file_read(const char* path, const char* tensor_name, void* dst, uint64_t dst_bytes, uint64_t* nelem_out)
{
    return guarded([&] {
        if (!path || !tensor_name) fail(ES_BAD_ARGUMENT, "weight file: null pointer");
        file_t      file(path, "rb");
        std::string name;
        uint64_t    nelem = 0;
        while (next_record(file.f, name, nelem)) {
            if (name == tensor_name) {
                if (nelem_out) *nelem_out = nelem;
                if (!dst) return;
                if (dst_bytes < nelem * 2) fail(ES_BAD_ARGUMENT, "weight file: destination too small");
                if (std::fread(dst, 2, nelem, file.f) != nelem) fail(ES_BAD_DESCRIPTOR, "weight file: truncated data");
                return;
            }
            if (std::fseek(file.f, (long)(nelem * 2), SEEK_CUR) != 0) fail(ES_BAD_DESCRIPTOR, "weight file: truncated data");
        }
        fail(ES_BAD_ARGUMENT, std::string("weight file: did not find \"") + tensor_name + "\"");
    });
}

int es_b200_weight_file_append(const char* path, const char* tensor_name, const void* f16_data, uint64_t nelem)
{
    return guarded([&] {
        if (!path || !tensor_name || (!f16_data && nelem)) fail(ES_BAD_ARGUMENT, "weight file: null pointer");
        size_t len = std::strlen(tensor_name);
        if (len > NAME_BYTES) fail(ES_BAD_ARGUMENT, "weight file: tensor names have at most 50 bytes");
        file_t file(path, "ab");
        char   raw[NAME_BYTES];
        std::memset(raw, ' ', NAME_BYTES);
        std::memcpy(raw, tensor_name, len);
        int64_t count = (int64_t)nelem;
        if (std::fwrite(raw, 1, NAME_BYTES, file.f) != NAME_BYTES || std::fwrite(&count, sizeof count, 1, file.f) != 1 ||
            std::fwrite(f16_data, 2, nelem, file.f) != nelem)
            fail(ES_CUDA_ERROR, "weight file: write failed");
    });
}

} // extern "C"
