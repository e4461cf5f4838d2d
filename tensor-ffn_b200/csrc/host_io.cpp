#include "host_io.h"
#include "json_lite.h"
#include <algorithm>
#include <cstring>
#include <dirent.h>
#include <fcntl.h>
#include <fstream>
#include <sstream>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace tffn {

std::string read_text_file(const std::string& path, bool* ok) {
    std::ifstream f(path, std::ios::binary);
    if (!f) {
        if (ok) *ok = false;
        return std::string();
    }
    std::ostringstream ss;
    ss << f.rdbuf();
    if (ok) *ok = true;
    return ss.str();
}

static int first_int(const JsonValue& j, const char* key, int def) {
    const JsonValue* v = j.find(key);
    if (!v) return def;
    if (v->is_array() && !v->arr.empty() && v->arr[0].is_number()) return (int)v->arr[0].as_int();
    if (v->is_number()) return (int)v->as_int();
    return def;
}

Config read_config(const std::string& dir) {
    bool ok;
    std::string text = read_text_file(dir + "/config.json", &ok);
    if (!ok) throw Error(kErrIO, "Cannot open " + dir + "/config.json");
    JsonValue j;
    try {
        j = json_parse(text);
    } catch (const std::exception& e) {
        throw Error(kErrFormat, dir + "/config.json: " + e.what());
    }
    Config c;
    c.hidden_size = (int)j.value_int("hidden_size", 896);
    c.intermediate_size = (int)j.value_int("intermediate_size", 4864);
    c.num_layers = (int)j.value_int("num_hidden_layers", 24);
    c.num_heads = (int)j.value_int("num_attention_heads", 14);
    c.num_kv_heads = (int)j.value_int("num_key_value_heads", 2);
    c.vocab_size = (int)j.value_int("vocab_size", 151936);
    c.max_seq_len = (int)j.value_int("max_position_embeddings", 131072);
    c.rms_norm_eps = (float)j.value_double("rms_norm_eps", 1e-6);
    c.rope_theta = (float)j.value_double("rope_theta", 1e6);
    c.tie_embeddings = j.value_bool("tie_word_embeddings", true);
    c.eos_token_id = first_int(j, "eos_token_id", 151645);
    c.bos_token_id = first_int(j, "bos_token_id", 151643);
    if (c.hidden_size <= 0 || c.num_heads <= 0 || c.num_kv_heads <= 0 || c.num_layers <= 0 ||
        c.intermediate_size <= 0 || c.vocab_size <= 0)
        throw Error(kErrFormat, "config.json: non-positive dimension");
    if (c.hidden_size % c.num_heads != 0 || c.num_heads % c.num_kv_heads != 0)
        throw Error(kErrFormat, "config.json: heads do not divide hidden size / kv heads do not divide heads");
    c.head_dim = c.hidden_size / c.num_heads;
    return c;
}

TpPartition tp_partition(const Config& c, int rank, int size) {
    if (size < 1 || rank < 0 || rank >= size) throw Error(kErrInvalid, "tensor-parallel rank / size out of range");
    TpPartition p;
    p.tp_rank = rank;
    p.tp_size = size;
    const int nh = c.num_heads, nkv = c.num_kv_heads, G = nh / nkv;
    if (size <= nkv) {
        if (nkv % size != 0) throw Error(kErrUnsupported, "tensor parallel: the kv heads do not divide among the ranks");
        p.n_kv_heads = nkv / size;
        p.kv_head0 = rank * p.n_kv_heads;
        p.q_head0 = p.kv_head0 * G;
        p.n_q_heads = p.n_kv_heads * G;
    } else {
        if (size % nkv != 0) throw Error(kErrUnsupported, "tensor parallel: the ranks do not divide among the kv heads");
        const int R = size / nkv, sub = rank % R;  // R ranks share kv head rank / R
        if (R > G) throw Error(kErrUnsupported, "tensor parallel: more ranks per kv head than query heads in its group");
        p.n_kv_heads = 1;
        p.kv_head0 = rank / R;
        const int a = G * sub / R, b = G * (sub + 1) / R;
        p.q_head0 = p.kv_head0 * G + a;
        p.n_q_heads = b - a;
    }
    if (c.intermediate_size % 64 != 0 && size > 1)
        throw Error(kErrUnsupported, "tensor parallel: the intermediate size must be a multiple of 64");
    const int iu = c.intermediate_size / 64;
    if (size > 1 && iu < size) throw Error(kErrUnsupported, "tensor parallel: intermediate size too small for this many ranks");
    p.i0 = size > 1 ? (int)((long long)iu * rank / size) * 64 : 0;
    p.n_i = size > 1 ? (int)((long long)iu * (rank + 1) / size) * 64 - p.i0 : c.intermediate_size;
    if (size > 1 && c.vocab_size % 8 != 0) throw Error(kErrUnsupported, "tensor parallel: the vocabulary size must be a multiple of 8");
    const int vu = c.vocab_size / 8;
    p.v0 = size > 1 ? (int)((long long)vu * rank / size) * 8 : 0;
    p.n_v = size > 1 ? (int)((long long)vu * (rank + 1) / size) * 8 - p.v0 : c.vocab_size;
    return p;
}

// ---------------------------------------------------------------- safetensors
static void* map_file(const std::string& path, size_t* size, int* fd_out) {
    int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw Error(kErrIO, "Cannot open " + path);
    struct stat st;
    if (fstat(fd, &st) != 0) {
        ::close(fd);
        throw Error(kErrIO, "Cannot stat " + path);
    }
    *size = (size_t)st.st_size;
    void* p = nullptr;
    if (*size > 0) {
        p = mmap(nullptr, *size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (p == MAP_FAILED) {
            ::close(fd);
            throw Error(kErrIO, "mmap failed for " + path);
        }
    }
    *fd_out = fd;
    return p;
}

static size_t dtype_size(const std::string& d) {
    if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    return 0;
}

SafeTensorsFile::SafeTensorsFile(const std::string& p) : path(p) {
    map_ = map_file(p, &size_, &fd_);
    auto bad = [&](const std::string& why) {
        if (map_) munmap(map_, size_);
        if (fd_ >= 0) ::close(fd_);
        map_ = nullptr;
        fd_ = -1;
        throw Error(kErrFormat, p + ": " + why);
    };
    if (size_ < 8) bad("file shorter than the 8-byte header length");
    const uint8_t* base = (const uint8_t*)map_;
    uint64_t hl;
    memcpy(&hl, base, 8);
    if (hl > size_ - 8) bad("header length exceeds file size");
    JsonValue header;
    try {
        header = json_parse((const char*)base + 8, (size_t)hl);
    } catch (const std::exception& e) {
        bad(std::string("header: ") + e.what());
    }
    if (!header.is_object()) bad("header is not an object");
    const uint8_t* data = base + 8 + hl;
    size_t data_size = size_ - 8 - (size_t)hl;
    for (auto& kv : header.obj) {
        if (kv.first == "__metadata__") continue;
        const JsonValue& v = kv.second;
        const JsonValue* dt = v.find("dtype");
        const JsonValue* sh = v.find("shape");
        const JsonValue* off = v.find("data_offsets");
        if (!dt || !dt->is_string() || !sh || !sh->is_array() || !off || !off->is_array() || off->arr.size() != 2)
            bad("malformed entry for " + kv.first);
        TensorInfo ti;
        ti.dtype = dt->str;
        size_t elems = 1;
        for (auto& d : sh->arr) {
            ti.shape.push_back(d.as_int());
            elems *= (size_t)d.as_int();
        }
        size_t s = (size_t)off->arr[0].as_int(), e = (size_t)off->arr[1].as_int();
        if (e < s || e > data_size) bad("data_offsets out of range for " + kv.first);
        size_t ds = dtype_size(ti.dtype);
        if (ds == 0) bad("Unknown dtype: " + ti.dtype);
        if (elems * ds != e - s) bad("shape and data_offsets disagree for " + kv.first);
        ti.data = data + s;
        ti.nbytes = e - s;
        tensors.emplace(kv.first, std::move(ti));
    }
}

SafeTensorsFile::~SafeTensorsFile() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
}

SafeTensorsDir::SafeTensorsDir(const std::string& dir) {
    DIR* d = opendir(dir.c_str());
    if (!d) throw Error(kErrIO, "Cannot open dir " + dir);
    std::vector<std::string> files;
    while (struct dirent* ent = readdir(d)) {
        std::string name = ent->d_name;
        const std::string suffix = ".safetensors";
        if (name.size() > suffix.size() && name.compare(name.size() - suffix.size(), suffix.size(), suffix) == 0)
            files.push_back(dir + "/" + name);
    }
    closedir(d);
    std::sort(files.begin(), files.end());
    if (files.empty()) throw Error(kErrIO, "No .safetensors file in " + dir);
    try {
        for (auto& f : files) shards_.push_back(new SafeTensorsFile(f));
    } catch (...) {
        for (auto* s : shards_) delete s;
        shards_.clear();
        throw;
    }
}
SafeTensorsDir::~SafeTensorsDir() {
    for (auto* s : shards_) delete s;
}
bool SafeTensorsDir::has(const std::string& name) const {
    for (auto* s : shards_)
        if (s->tensors.count(name)) return true;
    return false;
}
const TensorInfo& SafeTensorsDir::get(const std::string& name) const {
    for (auto* s : shards_) {
        auto it = s->tensors.find(name);
        if (it != s->tensors.end()) return it->second;
    }
    throw Error(kErrFormat, "Missing tensor: " + name);
}
const uint16_t* SafeTensorsDir::bf16(const std::string& name, size_t elems) const {
    const TensorInfo& ti = get(name);
    if (ti.dtype != "BF16") throw Error(kErrFormat, "Tensor " + name + " is " + ti.dtype + ", expected BF16");
    if (ti.nbytes != elems * 2) throw Error(kErrShape, "Size mismatch for " + name);
    return (const uint16_t*)ti.data;
}
size_t SafeTensorsDir::num_tensors() const {
    size_t n = 0;
    for (auto* s : shards_) n += s->tensors.size();
    return n;
}

// ---------------------------------------------------------------- expert .bin
ExpertFile::ExpertFile(const std::string& path) {
    map_ = map_file(path, &size_, &fd_);
    auto bad = [&](int code, const std::string& why) {
        if (map_) munmap(map_, size_);
        if (fd_ >= 0) ::close(fd_);
        map_ = nullptr;
        fd_ = -1;
        throw Error(code, path + ": " + why);
    };
    if (size_ < 20) bad(kErrFormat, "file shorter than the 20-byte header");
    memcpy(&hdr, map_, 20);
    if (hdr.magic != kExpertMagic) {
        char buf[96];
        snprintf(buf, sizeof buf, "Bad checkpoint magic: 0x%08x (expected 0x%08x)", hdr.magic, kExpertMagic);
        bad(kErrFormat, buf);
    }
    // The version word is read but not checked by the reference (inference/src/io/checkpoint.cpp:17);
    // the same holds here so that files from any trainer build load.
    unsigned __int128 need = (unsigned __int128)hdr.num_layers * 3u * hdr.hidden * hdr.intermediate * 4u + 20u;
    if (hdr.num_layers == 0 || hdr.hidden == 0 || hdr.intermediate == 0) bad(kErrFormat, "zero dimension in header");
    if (need > (unsigned __int128)size_) bad(kErrFormat, "file is truncated (fewer bytes than the header's shape needs)");
}
ExpertFile::~ExpertFile() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
}
const float* ExpertFile::matrix(int layer, int m) const {
    size_t per = matrix_elems();
    return (const float*)((const uint8_t*)map_ + 20) + ((size_t)layer * 3 + m) * per;
}

void write_expert(const std::string& path, uint32_t layers, uint32_t hidden, uint32_t inter,
                  const float* const* mats) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) throw Error(kErrIO, "Cannot save checkpoint " + path);
    uint32_t h[5] = {kExpertMagic, kExpertVersion, layers, hidden, inter};
    bool ok = fwrite(h, 4, 5, f) == 5;
    size_t n = (size_t)hidden * inter;
    for (uint32_t l = 0; ok && l < layers; ++l)
        for (int m = 0; ok && m < 3; ++m) ok = fwrite(mats[l * 3 + m], 4, n, f) == n;
    ok = (fclose(f) == 0) && ok;
    if (!ok) throw Error(kErrIO, "Short write to " + path);
}

// ---------------------------------------------------------------- tokenizer
void Tokenizer::load(const std::string& dir) {
    bool ok;
    std::string text = read_text_file(dir + "/tokenizer.json", &ok);
    if (!ok) throw Error(kErrIO, "Cannot open tokenizer.json");
    JsonValue j;
    try {
        j = json_parse(text);
    } catch (const std::exception& e) {
        throw Error(kErrFormat, std::string("tokenizer.json: ") + e.what());
    }
    const JsonValue* model = j.find("model");
    const JsonValue* vocab = model ? model->find("vocab") : nullptr;
    if (!vocab || !vocab->is_object()) throw Error(kErrFormat, "tokenizer.json: model.vocab missing");
    token_to_id_.reserve(vocab->obj.size() * 2);
    for (auto& kv : vocab->obj) {
        uint32_t id = (uint32_t)kv.second.as_int();
        token_to_id_[kv.first] = id;
        id_to_token_[id] = kv.first;
    }
    if (const JsonValue* ml = model->find("merges")) {
        for (auto& m : ml->arr) {
            std::string a, b;
            if (m.is_string()) {
                size_t sp = m.str.find(' ');
                if (sp == std::string::npos) continue;
                a = m.str.substr(0, sp);
                b = m.str.substr(sp + 1);
            } else if (m.is_array() && m.arr.size() == 2) {
                a = m.arr[0].str;
                b = m.arr[1].str;
            } else {
                continue;
            }
            auto ia = token_to_id_.find(a), ib = token_to_id_.find(b);
            if (ia == token_to_id_.end() || ib == token_to_id_.end()) continue;
            uint64_t key = (uint64_t)ia->second << 32 | ib->second;
            if (!merge_rank_.count(key)) merge_rank_[key] = (uint32_t)merges_.size();
            merges_.push_back({ia->second, ib->second});
        }
    }
    if (const JsonValue* at = j.find("added_tokens")) {
        for (auto& t : at->arr) {
            const JsonValue* c = t.find("content");
            const JsonValue* id = t.find("id");
            if (!c || !id) continue;
            token_to_id_[c->str] = (uint32_t)id->as_int();
            id_to_token_[(uint32_t)id->as_int()] = c->str;
            if (!c->str.empty()) added_.push_back(c->str);
        }
        std::sort(added_.begin(), added_.end(), [](const std::string& a, const std::string& b) { return a.size() > b.size(); });
    }
    std::string g = read_text_file(dir + "/generation_config.json", &ok);
    if (ok) {
        try {
            JsonValue gj = json_parse(g);
            eos_id = (uint32_t)first_int(gj, "eos_token_id", (int)eos_id);
            bos_id = (uint32_t)first_int(gj, "bos_token_id", (int)bos_id);
        } catch (const std::exception&) {
        }
    }
    pad_id = bos_id;
}

std::vector<uint32_t> Tokenizer::encode(const std::string& text) const {
    std::vector<uint32_t> ids;
    if (text.empty()) return ids;
    ids.reserve(text.size());
    for (unsigned char c : text) {
        auto it = token_to_id_.find(std::string(1, (char)c));
        if (it != token_to_id_.end()) {
            ids.push_back(it->second);
        } else {
            char hex[8];
            snprintf(hex, sizeof hex, "<0x%02X>", c);
            auto it2 = token_to_id_.find(hex);
            if (it2 != token_to_id_.end()) ids.push_back(it2->second);
        }
    }
    bool changed = true;
    while (changed && ids.size() > 1) {
        changed = false;
        uint32_t best_rank = UINT32_MAX;
        size_t best_pos = 0;
        for (size_t i = 0; i + 1 < ids.size(); ++i) {
            auto it = merge_rank_.find((uint64_t)ids[i] << 32 | ids[i + 1]);
            if (it != merge_rank_.end() && it->second < best_rank) {
                best_rank = it->second;
                best_pos = i;
            }
        }
        if (best_rank != UINT32_MAX) {
            auto& pr = merges_[best_rank];
            auto il = id_to_token_.find(pr.first), ir = id_to_token_.find(pr.second);
            if (il == id_to_token_.end() || ir == id_to_token_.end()) break;
            auto it = token_to_id_.find(il->second + ir->second);
            if (it != token_to_id_.end()) {
                ids[best_pos] = it->second;
                ids.erase(ids.begin() + best_pos + 1);
                changed = true;
            }
        }
    }
    return ids;
}

// ---------------------------------------------------------------- byte-level BPE as tokenizer.json specifies it
namespace {

#include "unicode_tables.inc"

bool in_ranges(const uint32_t (*r)[2], size_t n, uint32_t cp) {
    size_t lo = 0, hi = n;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (cp < r[mid][0]) hi = mid;
        else if (cp > r[mid][1]) lo = mid + 1;
        else return true;
    }
    return false;
}
bool is_letter(uint32_t cp) { return in_ranges(kUnicodeLetter, sizeof kUnicodeLetter / sizeof kUnicodeLetter[0], cp); }
bool is_number(uint32_t cp) { return in_ranges(kUnicodeNumber, sizeof kUnicodeNumber / sizeof kUnicodeNumber[0], cp); }
bool is_white(uint32_t cp) {
    for (uint32_t w : kUnicodeWhite)
        if (w == cp) return true;
    return false;
}
bool is_newline(uint32_t cp) { return cp == '\r' || cp == '\n'; }

// GPT-2's bytes_to_unicode: printable Latin-1 bytes stand for themselves, the other 68 bytes for U+0100 ...
struct ByteMap {
    uint32_t to_cp[256];
    std::unordered_map<uint32_t, uint8_t> to_byte;
    ByteMap() {
        int n = 0;
        for (int b = 0; b < 256; ++b) {
            const bool keep = (b >= 0x21 && b <= 0x7E) || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
            to_cp[b] = keep ? (uint32_t)b : (uint32_t)(256 + n++);
            to_byte[to_cp[b]] = (uint8_t)b;
        }
    }
};
const ByteMap& byte_map() {
    static const ByteMap m;
    return m;
}
void put_utf8(std::string& s, uint32_t cp) {
    if (cp < 0x80) {
        s += (char)cp;
    } else if (cp < 0x800) {
        s += (char)(0xC0 | (cp >> 6));
        s += (char)(0x80 | (cp & 0x3F));
    } else if (cp < 0x10000) {
        s += (char)(0xE0 | (cp >> 12));
        s += (char)(0x80 | ((cp >> 6) & 0x3F));
        s += (char)(0x80 | (cp & 0x3F));
    } else {
        s += (char)(0xF0 | (cp >> 18));
        s += (char)(0x80 | ((cp >> 12) & 0x3F));
        s += (char)(0x80 | ((cp >> 6) & 0x3F));
        s += (char)(0x80 | (cp & 0x3F));
    }
}
// code points of a UTF-8 string with the byte offset of each (a malformed byte counts as one code point)
void utf8_points(const std::string& s, std::vector<uint32_t>& cps, std::vector<size_t>& offs) {
    for (size_t i = 0; i < s.size();) {
        const unsigned char c = (unsigned char)s[i];
        int len = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1;
        if (i + len > s.size()) len = 1;
        uint32_t cp = len == 1 ? c : (c & (0xFF >> (len + 1)));
        for (int k = 1; k < len; ++k) {
            if (((unsigned char)s[i + k] & 0xC0) != 0x80) { len = 1; cp = c; break; }
            cp = (cp << 6) | ((unsigned char)s[i + k] & 0x3F);
        }
        cps.push_back(cp);
        offs.push_back(i);
        i += len;
    }
    offs.push_back(s.size());
}

// ---- NFC (Unicode Standard Annex 15), the normaliser Qwen2's tokenizer.json runs before the pre-tokenizer
uint32_t ccc_of(uint32_t cp) {
    size_t lo = 0, hi = sizeof kUnicodeCcc / sizeof kUnicodeCcc[0];
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (kUnicodeCcc[mid][0] < cp) lo = mid + 1;
        else if (kUnicodeCcc[mid][0] > cp) hi = mid;
        else return kUnicodeCcc[mid][1];
    }
    return 0;
}
constexpr uint32_t kSBase = 0xAC00, kLBase = 0x1100, kVBase = 0x1161, kTBase = 0x11A7;
constexpr uint32_t kLCount = 19, kVCount = 21, kTCount = 28, kNCount = kVCount * kTCount, kSCount = kLCount * kNCount;
void decompose_into(uint32_t cp, std::vector<uint32_t>& out) {
    if (cp >= kSBase && cp < kSBase + kSCount) {  // Hangul syllable: arithmetic
        const uint32_t sidx = cp - kSBase;
        out.push_back(kLBase + sidx / kNCount);
        out.push_back(kVBase + (sidx % kNCount) / kTCount);
        if (sidx % kTCount) out.push_back(kTBase + sidx % kTCount);
        return;
    }
    size_t lo = 0, hi = sizeof kUnicodeDecomp / sizeof kUnicodeDecomp[0];
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (kUnicodeDecomp[mid][0] < cp) lo = mid + 1;
        else if (kUnicodeDecomp[mid][0] > cp) hi = mid;
        else {
            decompose_into(kUnicodeDecomp[mid][1], out);  // decompositions nest a few levels at most
            if (kUnicodeDecomp[mid][2]) decompose_into(kUnicodeDecomp[mid][2], out);
            return;
        }
    }
    out.push_back(cp);
}
bool compose_pair(uint32_t a, uint32_t b, uint32_t* c) {
    if (a >= kLBase && a < kLBase + kLCount && b >= kVBase && b < kVBase + kVCount) {
        *c = kSBase + ((a - kLBase) * kVCount + (b - kVBase)) * kTCount;
        return true;
    }
    if (a >= kSBase && a < kSBase + kSCount && (a - kSBase) % kTCount == 0 && b > kTBase && b < kTBase + kTCount) {
        *c = a + (b - kTBase);
        return true;
    }
    size_t lo = 0, hi = sizeof kUnicodeCompose / sizeof kUnicodeCompose[0];
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        const uint32_t* e = kUnicodeCompose[mid];
        if (e[0] < a || (e[0] == a && e[1] < b)) lo = mid + 1;
        else if (e[0] > a || (e[0] == a && e[1] > b)) hi = mid;
        else {
            *c = e[2];
            return true;
        }
    }
    return false;
}
// NFC of well-formed UTF-8; text without a code point from U+0300 on is in NFC already and returned as it is,
// and so is text with a malformed byte (re-encoding would change its bytes).
std::string nfc_utf8(const std::string& s) {
    bool plain = true;
    for (unsigned char c : s)
        if (c >= 0xCC) { plain = false; break; }  // lead bytes below 0xCC encode code points below U+0300
    if (plain) return s;
    std::vector<uint32_t> cps;
    std::vector<size_t> offs;
    utf8_points(s, cps, offs);
    for (size_t i = 0; i < cps.size(); ++i) {
        const size_t len = offs[i + 1] - offs[i];
        const uint32_t cp = cps[i];
        const size_t want = cp < 0x80 ? 1 : cp < 0x800 ? 2 : cp < 0x10000 ? 3 : 4;
        if (len != want || cp > 0x10FFFF || (cp >= 0xD800 && cp < 0xE000)) return s;  // malformed or overlong
    }
    std::vector<uint32_t> d;
    d.reserve(cps.size() + 8);
    for (uint32_t cp : cps) decompose_into(cp, d);
    // canonical ordering: inside every run of non-starters, ascending combining class, stable
    for (size_t i = 1; i < d.size(); ++i) {
        const uint32_t cc = ccc_of(d[i]);
        if (cc == 0) continue;
        size_t j = i;
        while (j > 0) {
            const uint32_t pc = ccc_of(d[j - 1]);
            if (pc == 0 || pc <= cc) break;
            std::swap(d[j - 1], d[j]);
            --j;
        }
    }
    // canonical composition: a character combines with the last starter unless something between them blocks it
    std::vector<uint32_t> out;
    out.reserve(d.size());
    size_t starter = (size_t)-1;
    uint32_t last_cc = 0;
    for (uint32_t ch : d) {
        const uint32_t cc = ccc_of(ch);
        if (starter != (size_t)-1) {
            const bool adjacent = out.size() - 1 == starter;
            const bool blocked = !adjacent && (last_cc == 0 || last_cc >= cc);
            uint32_t c;
            if (!blocked && compose_pair(out[starter], ch, &c)) {
                out[starter] = c;
                continue;
            }
        }
        if (cc == 0) starter = out.size();
        out.push_back(ch);
        last_cc = cc;
    }
    std::string r;
    r.reserve(s.size());
    for (uint32_t cp : out) put_utf8(r, cp);
    return r;
}

// end (exclusive, in code points) of the pre-tokenizer match that starts at i: the pattern's alternatives in order
size_t pretok_match(const std::vector<uint32_t>& cp, size_t i) {
    const size_t n = cp.size();
    auto lower = [](uint32_t c) { return (c >= 'A' && c <= 'Z') ? c + 32 : c; };
    if (cp[i] == '\'' && i + 1 < n) {  // (?i:'s|'t|'re|'ve|'m|'ll|'d)
        const uint32_t a = lower(cp[i + 1]), b = i + 2 < n ? lower(cp[i + 2]) : 0;
        if (a == 's' || a == 't') return i + 2;
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e')) return i + 3;
        if (a == 'm') return i + 2;
        if (a == 'l' && b == 'l') return i + 3;
        if (a == 'd') return i + 2;
    }
    {  // [^\r\n\p{L}\p{N}]?\p{L}+
        size_t j = i;
        if (!is_letter(cp[j]) && !is_newline(cp[j]) && !is_number(cp[j]) && j + 1 < n && is_letter(cp[j + 1])) ++j;
        if (is_letter(cp[j])) {
            while (j < n && is_letter(cp[j])) ++j;
            return j;
        }
    }
    if (is_number(cp[i])) return i + 1;  // \p{N}
    {  //  ?[^\s\p{L}\p{N}]+[\r\n]*
        size_t j = i;
        auto other = [&](size_t k) { return !is_white(cp[k]) && !is_letter(cp[k]) && !is_number(cp[k]); };
        if (cp[j] == ' ' && j + 1 < n && other(j + 1)) ++j;
        if (other(j)) {
            while (j < n && other(j)) ++j;
            while (j < n && is_newline(cp[j])) ++j;
            return j;
        }
    }
    if (is_white(cp[i])) {
        size_t e = i;
        while (e < n && is_white(cp[e])) ++e;
        size_t last_nl = n;  // \s*[\r\n]+ : up to and including the last newline of the run
        for (size_t k = i; k < e; ++k)
            if (is_newline(cp[k])) last_nl = k;
        if (last_nl != n) return last_nl + 1;
        if (e == n) return e;      // \s+(?!\S) at the end of the text
        if (e - 1 > i) return e - 1;  // \s+(?!\S): leave the last blank to the next piece
        return e;                   // \s+
    }
    return i + 1;
}

}  // namespace

void Tokenizer::bpe_piece(const std::string& bytes, std::vector<uint32_t>& out) const {
    const ByteMap& bm = byte_map();
    std::vector<uint32_t> ids;
    ids.reserve(bytes.size());
    for (unsigned char b : bytes) {
        std::string ch;
        put_utf8(ch, bm.to_cp[b]);
        auto it = token_to_id_.find(ch);
        if (it == token_to_id_.end()) continue;  // a vocabulary without the byte alphabet: nothing stands for this byte
        ids.push_back(it->second);
    }
    while (ids.size() > 1) {
        uint32_t best_rank = UINT32_MAX;
        for (size_t i = 0; i + 1 < ids.size(); ++i) {
            auto it = merge_rank_.find((uint64_t)ids[i] << 32 | ids[i + 1]);
            if (it != merge_rank_.end() && it->second < best_rank) best_rank = it->second;
        }
        if (best_rank == UINT32_MAX) break;
        const auto& pr = merges_[best_rank];
        auto it = token_to_id_.find(id_to_token_.at(pr.first) + id_to_token_.at(pr.second));
        if (it == token_to_id_.end()) break;
        // every occurrence of the pair, left to right (what one pass of the standard algorithm does)
        std::vector<uint32_t> next;
        next.reserve(ids.size());
        for (size_t i = 0; i < ids.size();) {
            if (i + 1 < ids.size() && ids[i] == pr.first && ids[i + 1] == pr.second) {
                next.push_back(it->second);
                i += 2;
            } else {
                next.push_back(ids[i++]);
            }
        }
        ids.swap(next);
    }
    out.insert(out.end(), ids.begin(), ids.end());
}

std::vector<uint32_t> Tokenizer::encode_bpe(const std::string& text) const {
    std::vector<uint32_t> out;
    auto plain = [&](const std::string& raw) {
        if (raw.empty()) return;
        const std::string t = nfc_utf8(raw);  // tokenizer.json: normalizer NFC, then the Split pre-tokenizer
        std::vector<uint32_t> cps;
        std::vector<size_t> offs;
        utf8_points(t, cps, offs);
        for (size_t i = 0; i < cps.size();) {
            const size_t e = pretok_match(cps, i);
            bpe_piece(t.substr(offs[i], offs[e] - offs[i]), out);
            i = e;
        }
    };
    size_t start = 0, i = 0;
    while (i < text.size()) {  // added tokens (the ChatML markers ...) stand for themselves
        const std::string* hit = nullptr;
        for (const std::string& a : added_)
            if (text.compare(i, a.size(), a) == 0) { hit = &a; break; }
        if (!hit) { ++i; continue; }
        plain(text.substr(start, i - start));
        out.push_back(token_to_id_.at(*hit));
        i += hit->size();
        start = i;
    }
    plain(text.substr(start));
    return out;
}

std::string Tokenizer::decode_bpe(const std::vector<uint32_t>& ids) const {
    const ByteMap& bm = byte_map();
    std::string out;
    for (uint32_t id : ids) {
        auto it = id_to_token_.find(id);
        if (it == id_to_token_.end()) continue;
        const std::string& tok = it->second;
        if (std::find(added_.begin(), added_.end(), tok) != added_.end()) {
            out += tok;
            continue;
        }
        std::vector<uint32_t> cps;
        std::vector<size_t> offs;
        utf8_points(tok, cps, offs);
        for (uint32_t cp : cps) {
            auto b = bm.to_byte.find(cp);
            if (b != bm.to_byte.end()) out += (char)b->second;
        }
    }
    return out;
}

std::string Tokenizer::decode(const std::vector<uint32_t>& ids) const {
    std::string joined;
    for (uint32_t id : ids) {
        auto it = id_to_token_.find(id);
        if (it != id_to_token_.end()) joined += it->second;
    }
    std::string out;
    for (size_t i = 0; i < joined.size();) {
        if ((unsigned char)joined[i] == 0xC4 && i + 1 < joined.size() && (unsigned char)joined[i + 1] == 0xA0) {
            out += ' ';
            i += 2;
        } else {
            out += joined[i++];
        }
    }
    return out;
}

uint32_t Tokenizer::get_id(const std::string& token) const {
    auto it = token_to_id_.find(token);
    if (it != token_to_id_.end()) return it->second;
    fprintf(stderr, "Warning: special token '%s' not found in vocab.\n", token.c_str());
    return 0;
}

}  // namespace tffn
