// deepxIR host core — see core.hpp.
#include <cerrno>
#include <climits>

#include "core.hpp"
#include "fusion.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <cctype>
#include <iostream>
#include <sstream>

namespace dxh {

// ============================================================================================
// dtype codec
// ============================================================================================
namespace {
struct PrecName { uint16_t bit; const char *name; };
// order = the order precision_str lists the bits in (dtype.hpp:274-301)
const PrecName kPrecisions[] = {
    {P_F64, "float64"}, {P_F32, "float32"}, {P_F16, "float16"}, {P_BF16, "bfloat16"}, {P_F8E5M2, "float8e5m2"},
    {P_F8E4M3, "float8e4m3"}, {P_F4E2M1, "float4e2m1"}, {P_I64, "int64"}, {P_I32, "int32"}, {P_I16, "int16"},
    {P_I8, "int8"}, {P_I4, "int4"}, {P_BOOL, "bool"}, {P_STRING, "string"},
};
struct CatName { uint8_t bit; const char *name; };
// order of base_category_str (dtype.hpp:65-72)
const CatName kCategories[] = {{CAT_TENSOR, "tensor"}, {CAT_VECTOR, "vector"}, {CAT_VAR, "var"}, {CAT_LISTTENSOR, "listtensor"}};

void trim_spaces(std::string &s) {  // stdutil::trimspace: blanks only, not tabs (stdutil/string.cpp:6-10)
    size_t b = s.find_first_not_of(' ');
    if (b == std::string::npos) { s.clear(); return; }
    size_t e = s.find_last_not_of(' ');
    s = s.substr(b, e - b + 1);
}
void trim_chars(std::string &s, const char *chars) {  // stdutil::trim
    size_t b = s.find_first_not_of(chars);
    if (b == std::string::npos) { s.clear(); return; }
    size_t e = s.find_last_not_of(chars);
    s = s.substr(b, e - b + 1);
}
}  // namespace

uint8_t category_of(const std::string &text) {
    uint8_t out = CAT_UNKNOWN;
    size_t start = 0;
    while (true) {
        size_t bar = text.find('|', start);
        const std::string part = text.substr(start, bar == std::string::npos ? std::string::npos : bar - start);
        for (const auto &c : kCategories)
            if (part == c.name) out |= c.bit;
        if (bar == std::string::npos) break;
        start = bar + 1;
    }
    return out;
}

std::string category_str(uint8_t c) {
    std::string out;
    for (const auto &k : kCategories)
        if (c & k.bit) {
            if (!out.empty()) out += "|";
            out += k.name;
        }
    return out.empty() ? "unknown" : out;
}

uint16_t precision_of(const std::string &text) {
    // single names and the three group names only; anything else (including a|b lists) is "any"
    if (text == "any") return P_ANY;
    if (text == "int") return P_INT;
    if (text == "float") return P_FLOAT;
    if (text == "float8") return P_FLOAT8;
    for (const auto &p : kPrecisions)
        if (text == p.name) return p.bit;
    return P_ANY;
}

std::string precision_str(uint16_t p) {
    if (p == P_ANY) return "any";
    std::string out;
    for (const auto &k : kPrecisions)
        if (p & k.bit) {
            if (!out.empty()) out += "|";
            out += k.name;
        }
    return out.empty() ? "any" : out;
}

TypeDef typedef_of(const std::string &text) {
    TypeDef t;
    const size_t lt = text.find('<'), gt = text.find('>');
    if (lt == std::string::npos || gt == std::string::npos) {
        t.category = category_of(text);
        t.precision = P_ANY;
        return t;
    }
    t.category = category_of(text.substr(0, lt));
    t.precision = precision_of(text.substr(lt + 1, gt - lt - 1));
    return t;
}

std::string typedef_str(const TypeDef &t) { return category_str(t.category) + "<" + precision_str(t.precision) + ">"; }

int precision_bits(uint16_t p) {
    switch (p) {
        case P_F64: case P_I64: return 64;
        case P_F32: case P_I32: return 32;
        case P_F16: case P_BF16: case P_I16: return 16;
        case P_F8E5M2: case P_F8E4M3: case P_I8: case P_BOOL: return 8;
        default: return 0;
    }
}

int dx_code_of(uint16_t p) {
    switch (p) {
        case P_F64: return DX_F64;
        case P_F32: return DX_F32;
        case P_F16: return DX_F16;
        case P_BF16: return DX_BF16;
        case P_I64: return DX_I64;
        case P_I32: return DX_I32;
        case P_I16: return DX_I16;
        case P_I8: return DX_I8;
        case P_BOOL: return DX_BOOL;
        default: return -1;
    }
}
uint16_t precision_of_dx(int code) {
    static const uint16_t t[] = {P_F64, P_F32, P_F16, P_BF16, P_I64, P_I32, P_I16, P_I8, P_BOOL};
    return (code >= 0 && code < 9) ? t[code] : uint16_t(P_ANY);
}

bool is_float_text(const std::string &s) {
    try { (void)std::stof(s); return true; } catch (...) { return false; }
}
bool is_integer_text(const std::string &s) {
    try { (void)std::stoi(s); return true; } catch (...) { return false; }
}

// ============================================================================================
// shape
// ============================================================================================
void Shape::set(const std::vector<int64_t> &s) {
    shape = s;
    strides.assign(s.size(), 1);
    for (int i = int(s.size()) - 2; i >= 0; --i) strides[i] = strides[i + 1] * s[i + 1];
    size = s.empty() ? 0 : strides[0] * s[0];
}

std::string Shape::to_yaml() const {
    std::ostringstream o;
    o << "dtype: " << precision_str(dtype) << "\n";
    o << "dim: " << dim() << "\n";
    o << "shape:\n";
    for (auto v : shape) o << "  - " << v << "\n";
    o << "stride:\n";
    for (auto v : strides) o << "  - " << v << "\n";
    o << "size: " << size;
    return o.str();
}

Shape Shape::from_yaml(const std::string &text) {
    // The document has five flat keys; sequences come in block ("- 3") or flow ("[3, 4]") style.
    std::unordered_map<std::string, std::string> scalars;
    std::unordered_map<std::string, std::vector<int64_t>> seqs;
    std::istringstream in(text);
    std::string line, current;
    auto parse_flow = [](std::string v) {
        std::vector<int64_t> out;
        trim_chars(v, " []");
        std::istringstream ss(v);
        std::string item;
        while (std::getline(ss, item, ',')) {
            trim_chars(item, " ");
            if (!item.empty()) out.push_back(std::stoll(item));
        }
        return out;
    };
    while (std::getline(in, line)) {
        if (!line.empty() && line.back() == '\r') line.pop_back();
        std::string t = line;
        trim_chars(t, " ");
        if (t.empty() || t[0] == '#') continue;
        if (t[0] == '-') {
            std::string v = t.substr(1);
            trim_chars(v, " ");
            if (current.empty()) throw std::runtime_error("Shape::fromYaml: sequence item without a key");
            seqs[current].push_back(std::stoll(v));
            continue;
        }
        const size_t colon = t.find(':');
        if (colon == std::string::npos) throw std::runtime_error("Shape::fromYaml: cannot parse line: " + t);
        std::string key = t.substr(0, colon), val = t.substr(colon + 1);
        trim_chars(key, " ");
        trim_chars(val, " ");
        current = key;
        if (val.empty()) { seqs[key]; continue; }
        if (val[0] == '[') seqs[key] = parse_flow(val);
        else {
            trim_chars(val, "'\"");
            scalars[key] = val;
        }
    }
    if (!scalars.count("dtype") || !seqs.count("shape")) throw std::runtime_error("Shape::fromYaml: dtype or shape missing");
    Shape s(seqs["shape"]);
    s.dtype = precision_of(scalars["dtype"]);
    if (seqs.count("stride") && seqs["stride"] != s.strides) throw std::runtime_error("Shape::fromYaml: strides mismatch");
    if (scalars.count("size") && std::stoll(scalars["size"]) != s.size) throw std::runtime_error("Shape::fromYaml: size mismatch");
    return s;
}

std::vector<int64_t> transpose_shape(const std::vector<int64_t> &shape, const std::vector<int> &order) {
    if (order.size() != shape.size())
        throw std::invalid_argument("dimOrder size does not match the number of dimensions in the TensorCPU.");
    std::vector<int64_t> out(shape.size());
    for (size_t i = 0; i < order.size(); ++i) {
        if (order[i] < 0 || order[i] >= int(shape.size())) throw std::invalid_argument("dimOrder entry out of range");
        out[i] = shape[order[i]];
    }
    return out;
}

std::vector<int64_t> broadcast_shape(const std::vector<int64_t> &a, const std::vector<int64_t> &b) {
    const size_t n = std::max(a.size(), b.size());
    std::vector<int64_t> out(n);
    for (size_t i = 1; i <= n; ++i) {
        const int64_t x = i <= a.size() ? a[a.size() - i] : 1, y = i <= b.size() ? b[b.size() - i] : 1;
        if (x != y && x != 1 && y != 1) return {};
        out[n - i] = std::max(x, y);
    }
    return out;
}

std::vector<int64_t> indexselect_shape(const std::vector<int64_t> &in, const std::vector<int64_t> &idx, int axis) {
    std::vector<int64_t> out(in.begin(), in.begin() + axis);
    out.insert(out.end(), idx.begin(), idx.end());
    out.insert(out.end(), in.begin() + axis + 1, in.end());
    return out;
}

std::vector<int64_t> repeat_shape(const std::vector<int64_t> &src, const std::vector<int64_t> &repeats) {
    if (src.size() != repeats.size()) throw std::invalid_argument("Shape and repeats must have the same number of dimensions");
    std::vector<int64_t> out(src.size());
    for (size_t i = 0; i < src.size(); ++i) out[i] = src[i] * repeats[i];
    return out;
}

std::vector<int> checked_dims(const std::vector<int64_t> &shape, const std::vector<int> &dims) {
    std::vector<int> out;
    const int n = int(shape.size());
    if (dims.empty()) {
        for (int i = 0; i < n; ++i) out.push_back(i);
    } else {
        for (int d : dims) {
            if (d < 0) d += n;
            if (d >= n || d < 0) throw TensorShapeError("Dimension out of range in sum");
            out.push_back(d);
        }
    }
    std::sort(out.begin(), out.end());
    out.erase(std::unique(out.begin(), out.end()), out.end());
    return out;
}

std::vector<int64_t> reduced_shape(const std::vector<int64_t> &shape, const std::vector<int> &checked, bool keepdims) {
    std::vector<char> red(shape.size(), 0);
    for (int d : checked) red[d] = 1;
    std::vector<int64_t> out;
    for (size_t i = 0; i < shape.size(); ++i) {
        if (!red[i]) out.push_back(shape[i]);
        else if (keepdims) out.push_back(1);
    }
    if (out.empty()) out.push_back(1);
    return out;
}

std::vector<int64_t> matmul_shape(const std::vector<int64_t> &a, const std::vector<int64_t> &b) {
    if (a.size() < 2 || b.size() < 2) throw std::invalid_argument("A and B must >= 2D tensors");
    if (a[a.size() - 1] != b[b.size() - 2]) throw std::invalid_argument("A[-1] must be equal to B[-2]");
    std::vector<int64_t> out = a;
    out.back() = b.back();
    return out;
}

bool check_matmul_shape(const std::vector<int64_t> &a, const std::vector<int64_t> &b) {
    if (a.size() < 2 || b.size() < 2) return false;
    if (a[a.size() - 1] != b[b.size() - 2]) return false;
    if (a.size() != b.size()) return false;
    for (size_t i = 0; i + 2 < a.size(); ++i)
        if (a[i] != b[i]) return false;
    return true;
}

// ============================================================================================
// tensors and the store
// ============================================================================================
Tensor::~Tensor() {
    if (ready_event) {
        cudaEventSynchronize(static_cast<cudaEvent_t>(ready_event));  // a copy into this storage may still be running
        cudaEventDestroy(static_cast<cudaEvent_t>(ready_event));
    }
    if (data && pool) dx_pool_free(pool, data);
    data = nullptr;
}

Mem::Mem(int device, size_t pool_limit_bytes) : device_(device) {
    pool_ = dx_pool_create(device, pool_limit_bytes);
    if (!pool_) throw std::runtime_error(std::string("cannot create the device pool: ") + dx_last_error());
    cudaSetDevice(device);
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        s = nullptr;  // fall back to the default stream
    }
    stream_ = s;
}

void *Mem::copy_stream() {
    if (!copy_stream_) {
        cudaStream_t s = nullptr;
        if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) throw std::runtime_error("cannot create the copy stream");
        copy_stream_ = s;
        cudaEvent_t e = nullptr;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) throw std::runtime_error("cannot create an event");
        order_event_ = e;
    }
    return copy_stream_;
}

void Mem::upload_async(Tensor &t, const void *host, size_t bytes) {
    cudaStream_t cs = static_cast<cudaStream_t>(copy_stream()), st = static_cast<cudaStream_t>(stream_);
    // the copy must not overtake earlier ops that still read or write this storage
    cudaEventRecord(static_cast<cudaEvent_t>(order_event_), st);
    cudaStreamWaitEvent(cs, static_cast<cudaEvent_t>(order_event_), 0);
    const cudaError_t e = cudaMemcpyAsync(t.data, host, bytes, cudaMemcpyHostToDevice, cs);
    if (e != cudaSuccess) throw std::runtime_error(std::string("host to device copy failed: ") + cudaGetErrorString(e));
    if (!t.ready_event) {
        cudaEvent_t ev = nullptr;
        if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) throw std::runtime_error("cannot create an event");
        t.ready_event = ev;
    }
    cudaEventRecord(static_cast<cudaEvent_t>(t.ready_event), cs);
    t.upload_in_flight = true;
}

void Mem::wait_ready(Tensor &t) {
    if (!t.upload_in_flight) return;
    cudaStreamWaitEvent(static_cast<cudaStream_t>(stream_), static_cast<cudaEvent_t>(t.ready_event), 0);
    t.upload_in_flight = false;
}

Mem::~Mem() {
    tensors_.clear();
    if (copy_stream_) {
        cudaStreamSynchronize(static_cast<cudaStream_t>(copy_stream_));
        cudaStreamDestroy(static_cast<cudaStream_t>(copy_stream_));
        cudaEventDestroy(static_cast<cudaEvent_t>(order_event_));
    }
    if (scratch_) dx_pool_free(pool_, scratch_);
    if (stream_) {
        cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
        cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
    }
    dx_pool_destroy(pool_);
}

TensorPtr Mem::new_tensor(const std::string &name, uint16_t precision, const std::vector<int64_t> &shape) {
    if (dx_code_of(precision) < 0) throw std::runtime_error("newtensor: unsupported precision");
    for (auto d : shape)
        if (d < 0) throw std::invalid_argument("newtensor: negative extent");
    auto t = std::make_shared<Tensor>();
    if (should_partition(shape, precision_bits(precision) / 8, shard)) {
        const RowBlock b = row_block(shape[0], shard.rank, shard.world);
        std::vector<int64_t> local = shape;
        local[0] = b.rows;
        t->shape.set(local);
        t->global_rows = shape[0];
        t->row0 = b.row0;
    } else {
        t->shape.set(shape);
    }
    t->shape.dtype = precision;
    t->pool = pool_;
    t->device = device_;
    const int64_t bytes = t->shape.bytes();
    t->data = dx_pool_alloc(pool_, size_t(std::max<int64_t>(bytes, 1)));
    if (!t->data) throw std::runtime_error(std::string("newtensor: ") + dx_last_error());
    add_tensor(name, t);
    return t;
}

void Mem::add_tensor(const std::string &name, TensorPtr t) {
    if (tensors_.count(name)) {
        std::cerr << "tensor already exists: " << name << std::endl;
        return;
    }
    tensors_[name] = std::move(t);
}

TensorPtr Mem::get_tensor(const std::string &name) const {
    auto it = tensors_.find(name);
    if (it == tensors_.end()) throw std::runtime_error("tensor not found: " + name);
    return it->second;
}

void Mem::rename_tensor(const std::string &old_name, const std::string &new_name) {
    auto it = tensors_.find(old_name);
    if (it == tensors_.end()) throw std::runtime_error("tensor not found: " + old_name);
    TensorPtr t = it->second;
    tensors_.erase(it);
    tensors_[new_name] = t;
}

const ArgValue *Mem::get_arg(const std::string &name) const {
    auto it = args_.find(name);
    if (it == args_.end()) {
        std::cerr << "arg not found: " << name << std::endl;
        return nullptr;
    }
    return &it->second;
}

void Mem::flush_comm() {
    if (!shard.comm) return;
    if (dx_comm_allreduce_finish(shard.comm, stream_) != DX_OK) throw std::runtime_error(dx_last_error());
}

bool Mem::comm_pending_in(const void *p, size_t bytes) const {
    void *buf = nullptr;
    if (!shard.comm || !dx_comm_pending(shard.comm, &buf)) return false;
    const char *lo = static_cast<const char *>(p);
    return static_cast<const char *>(buf) >= lo && static_cast<const char *>(buf) < lo + (bytes ? bytes : 1);
}

void *Mem::scratch(size_t bytes) {
    if (bytes <= scratch_bytes_) return scratch_;
    if (capturing) throw std::runtime_error("the reduce workspace would have to grow while a program is being captured");
    ++scratch_generation_;
    if (scratch_) dx_pool_free(pool_, scratch_);
    scratch_bytes_ = std::max(bytes, size_t(1) << 20);
    scratch_ = dx_pool_alloc(pool_, scratch_bytes_);
    if (!scratch_) {
        scratch_bytes_ = 0;
        throw std::runtime_error(std::string("reduce workspace: ") + dx_last_error());
    }
    return scratch_;
}

std::vector<std::string> Mem::tensor_names() const {
    std::vector<std::string> out;
    for (auto &kv : tensors_) out.push_back(kv.first);
    std::sort(out.begin(), out.end());
    return out;
}

// ============================================================================================
// IR
// ============================================================================================
void Param::parse(const std::string &text) {
    const size_t colon = text.find(':');
    std::string type, value;
    if (colon != std::string::npos) {
        type = text.substr(0, colon);
        value = text.substr(colon + 1);
        trim_spaces(type);
    } else value = text;
    trim_spaces(value);
    // no explicit type: the text itself is looked up as a type name (unknown category, any precision)
    dtype = typedef_of(type.empty() ? value : type);
    textvalue = value;
}

void Metadata::parse(const std::string &meta) {
    if (meta.empty()) return;
    using std::chrono::system_clock;
    // whitespace-separated key=value tokens; a token without '=' is ignored; the last value of a key wins
    // (plain scanning: this runs once per IR line, and string streams cost more than the rest of the parse)
    size_t pos = 0;
    const size_t n = meta.size();
    while (pos < n) {
        while (pos < n && std::isspace(static_cast<unsigned char>(meta[pos]))) ++pos;
        size_t end = pos;
        while (end < n && !std::isspace(static_cast<unsigned char>(meta[end]))) ++end;
        if (end > pos) {
            const size_t eq = meta.find('=', pos);
            if (eq != std::string::npos && eq < end) {
                const std::string key = meta.substr(pos, eq - pos), val = meta.substr(eq + 1, end - eq - 1);
                if (key == "id") id = std::stoi(val);
                else if (key == "author") author = val;
                else if (key == "created_at") created_at = system_clock::from_time_t(time_t(std::stod(val)));
                else if (key == "sent_at") sent_at = system_clock::from_time_t(time_t(std::stod(val)));
                else if (key == "recv_at") recv_at = system_clock::from_time_t(time_t(std::stod(val)));
                else if (key == "benchmark.repeat") benchmark_repeat = std::stoi(val);
            }
        }
        pos = end;
    }
}

namespace {
std::vector<Param> parse_params(const std::string &list) {
    std::vector<Param> out;
    size_t pos = 0;
    while (pos <= list.size()) {
        size_t comma = list.find(',', pos);
        if (comma == std::string::npos) comma = list.size();
        std::string item = list.substr(pos, comma - pos);
        trim_spaces(item);
        if (!item.empty()) {
            out.emplace_back();
            out.back().parse(item);
        }
        pos = comma + 1;
    }
    return out;
}
// text between the first '(' and the last ')', if both exist
bool inside_parens(const std::string &s, std::string *inner) {
    const size_t open = s.find('('), close = s.rfind(')');
    if (open == std::string::npos || close == std::string::npos) return false;
    *inner = (close > open) ? s.substr(open + 1, close - open - 1) : std::string();
    return true;
}
}  // namespace

void TF::parse(const std::string &text) {
    const size_t meta_pos = text.find("//");
    const std::string body = text.substr(0, meta_pos);
    const std::string meta = meta_pos == std::string::npos ? std::string() : text.substr(meta_pos + 2);
    const size_t arrow = body.find("->");
    if (arrow == std::string::npos) throw std::runtime_error("Invalid IR format: missing arrow");
    std::string in_part = body.substr(0, arrow), out_part = body.substr(arrow + 2);
    // op name ends at the first '(' if that comes before the first blank, else at the first blank
    const size_t blank = in_part.find(' '), paren = in_part.find('(');
    size_t name_end;
    if (paren != std::string::npos && (blank == std::string::npos || paren < blank)) name_end = paren;
    else name_end = blank != std::string::npos ? blank : in_part.size();
    name = in_part.substr(0, name_end);
    in_part = in_part.substr(name_end);
    std::string inner;
    if (inside_parens(in_part, &inner)) in_part = inner;
    else if (!in_part.empty() && in_part[0] == ' ') in_part = in_part.substr(1);
    if (inside_parens(out_part, &inner)) out_part = inner;
    args = parse_params(in_part);
    returns = parse_params(out_part);
    metadata.parse(meta);
}

std::string TF::to_string() const {
    std::string s = name + "(";
    for (size_t i = 0; i < args.size(); ++i) s += (i ? ", " : "") + args[i].to_string();
    s += ")->(";
    for (size_t i = 0; i < returns.size(); ++i) s += (i ? ", " : "") + returns[i].to_string();
    return s + ")";
}

const Param &TF::param(int idx, bool from_args) const {
    const std::vector<Param> &v = from_args ? args : returns;
    if (idx < 0) idx += int(v.size());
    if (idx < 0 || idx >= int(v.size())) throw std::invalid_argument("Invalid argument index");
    return v[idx];
}

bool TF::var_bool(int idx, bool from_args) const {
    std::string v = param(idx, from_args).textvalue;
    std::string low = v;
    std::transform(low.begin(), low.end(), low.begin(), [](unsigned char c) { return std::tolower(c); });
    if (low == "true") return true;
    if (low == "false") return false;
    throw std::invalid_argument("Invalid bool value:" + v);
}

float TF::var_f32(int idx, const Mem &mem, bool from_args) const {
    const std::string &text = param(idx, from_args).textvalue;
    if (is_float_text(text)) return std::stof(text);
    const ArgValue *a = mem.get_arg(text);  // a named arg set earlier with argset
    if (!a) return 0.f;
    if (auto p = std::get_if<int>(a)) return float(*p);
    if (auto p = std::get_if<float>(a)) return *p;
    if (auto p = std::get_if<double>(a)) return float(*p);
    return 0.f;
}

std::vector<std::string> TF::vector_text(int idx, bool from_args) const {
    std::string text = param(idx, from_args).textvalue;
    trim_chars(text, "[]");
    if (text.empty()) throw std::invalid_argument("Invalid argument index");
    std::vector<std::string> out;
    std::istringstream ss(text);
    std::string item;
    while (std::getline(ss, item, ' ')) out.push_back(item);
    return out;
}

// The reference converts every item with to<int> = int(std::stof(text)) (dtype.hpp:15-25), which rounds
// extents above 2^24 and is undefined from 2^31 on.  Text that is a plain integer is read exactly here
// (the two agree wherever the reference's result is defined and exact); text with a '.', an exponent or
// anything else still goes through std::stof.  Values outside the int64 range, or not finite, are refused.
std::vector<int64_t> TF::vector_i64(int idx, bool from_args) const {
    std::vector<int64_t> out;
    for (const auto &item : vector_text(idx, from_args)) {
        const char *b = item.c_str();
        char *end = nullptr;
        errno = 0;
        const long long v = std::strtoll(b, &end, 10);
        if (end != b && *end == 0) {
            if (errno == ERANGE) throw std::invalid_argument("integer out of range: " + item);
            out.push_back(v);
            continue;
        }
        const float f = std::stof(item);
        if (!(f > -9.2e18f && f < 9.2e18f)) throw std::invalid_argument("integer out of range: " + item);
        out.push_back(int64_t(f));
    }
    return out;
}

std::vector<int> TF::vector_int(int idx, bool from_args) const {
    std::vector<int> out;
    for (int64_t v : vector_i64(idx, from_args)) {
        if (v < INT32_MIN || v > INT32_MAX) throw std::invalid_argument("integer out of range: " + std::to_string(v));
        out.push_back(int(v));
    }
    return out;
}

bool TF::check_tensors(const std::vector<std::string> &names, const Mem &mem, std::string &error) const {
    for (const auto &n : names)
        if (!mem.exists_tensor(n)) {
            error = "tensor not found: " + n;
            return false;
        }
    return true;
}

std::string OpResp::to_string() const {
    using namespace std::chrono;
    std::ostringstream s;
    s << id << " " << result << "// recv_at=" << duration_cast<milliseconds>(recv_at.time_since_epoch()).count()
      << " start_at=" << duration_cast<milliseconds>(start_at.time_since_epoch()).count()
      << " finish_at=" << duration_cast<milliseconds>(finish_at.time_since_epoch()).count();
    if (!message.empty()) s << " " << message;
    return s.str();
}

// ============================================================================================
// registry
// ============================================================================================
void TfFactory::add_tf(std::shared_ptr<TF> tf) {
    auto it = families_.find(tf->name);
    if (it == families_.end()) {
        order_.push_back(tf->name);
        it = families_.emplace(tf->name, Family{}).first;
    }
    Family &fam = it->second;
    Author *author = nullptr;
    for (auto &a : fam.authors)
        if (a.name == tf->metadata.author) author = &a;
    if (!author) {
        fam.authors.push_back(Author{tf->metadata.author, {}});
        author = &fam.authors.back();
    }
    author->tfs.push_back(std::move(tf));
    ++count_;
}

std::shared_ptr<TF> TfFactory::get_tf(const TF &call, std::string *why) const {
    auto fam = families_.find(call.name);
    if (fam == families_.end()) {
        if (why) *why = "<op> " + call.name + " not found";
        return nullptr;
    }
    const Author *author = nullptr;
    for (const auto &a : fam->second.authors)
        if (a.name == call.metadata.author) author = &a;
    if (!author) author = &fam->second.authors.front();  // unknown author: first one registered
    for (const auto &tf : author->tfs) {
        if (tf->args.size() != call.args.size() || tf->returns.size() != call.returns.size()) continue;
        bool ok = true;
        for (size_t i = 0; ok && i < call.args.size(); ++i) ok = call.args[i].dtype.match(tf->args[i].dtype);
        for (size_t i = 0; ok && i < call.returns.size(); ++i) ok = call.returns[i].dtype.match(tf->returns[i].dtype);
        if (!ok) continue;
        auto cloned = tf->clone();
        cloned->metadata = call.metadata;
        return cloned;
    }
    if (why) {
        std::string msg = "<op> " + call.name + " " + call.to_string() + " not found; supported dtypes:";
        for (const auto &tf : author->tfs) {
            msg += " (";
            for (size_t i = 0; i < tf->args.size(); ++i) msg += (i ? ", " : "") + typedef_str(tf->args[i].dtype);
            msg += ")->(";
            for (size_t i = 0; i < tf->returns.size(); ++i) msg += (i ? ", " : "") + typedef_str(tf->returns[i].dtype);
            msg += ")";
        }
        *why = msg;
    }
    return nullptr;
}

namespace {
std::string escape_markdown(const std::string &s) {  // stdutil/string.cpp:18-53
    std::string out;
    for (char c : s) {
        switch (c) {
            case '\\': out += "\\\\"; break;
            case '"': out += "\\\""; break;
            case '\'': out += "\\'"; break;
            case '\n': out += "\\n"; break;
            case '\t': out += "\\t"; break;
            case '\r': out += "\\r"; break;
            case '\b': out += "\\b"; break;
            case '\f': out += "\\f"; break;
            default: out += c;
        }
    }
    return out;
}
}  // namespace

std::string TfFactory::print_markdown(const std::string &executor_name) const {
    std::ostringstream ss;
    ss << "## " << executor_name << " 支持算子列表 \n\n";
    ss << "本页面由 `executor/" << executor_name << " 生成，请勿手动修改 \n\n";
    std::vector<std::string> types;
    std::unordered_map<std::string, std::vector<std::shared_ptr<TF>>> by_type;
    for (const auto &name : order_)
        for (const auto &a : families_.at(name).authors)
            for (const auto &tf : a.tfs) {
                if (!by_type.count(tf->tftype)) types.push_back(tf->tftype);
                by_type[tf->tftype].push_back(tf);
            }
    for (const auto &type : types) {
        ss << "### " << type << "\n\n";
        ss << "| Operation | Author |  Math Formula | IR Instruction |\n";
        ss << "|-----------|--------|--------------|----------------|\n";
        for (const auto &tf : by_type[type]) {
            ss << "| " << tf->name << " | " << (tf->metadata.author.empty() ? " none " : tf->metadata.author) << " | "
               << tf->math_formula() << " | " << escape_markdown(tf->to_string()) << " |\n";
        }
        ss << "\n";
    }
    return ss.str();
}

// ============================================================================================
// executor
// ============================================================================================
Executor::Executor(int device, size_t pool_limit_bytes) : mem_(device, pool_limit_bytes) {
    register_all(factory_);
    register_fused(factory_);
}

OpResp Executor::run(const TF &call) {
    OpResp resp;
    resp.id = call.metadata.id;
    resp.recv_at = call.metadata.recv_at;
    resp.start_at = std::chrono::system_clock::now();
    if (ir_log) std::cout << "~" << call.to_string() << std::endl;
    std::string why;
    auto tf = factory_.get_tf(call, &why);
    if (!tf) {
        std::cerr << why << std::endl;
        resp.error("op" + call.name + " not found");
        return resp;
    }
    tf->name = call.name;
    tf->args = call.args;
    tf->returns = call.returns;
    std::lock_guard<std::mutex> lk(mu_);
    cudaSetDevice(mem_.device());
    resp.start_at = std::chrono::system_clock::now();
    std::string message;
    int rc = 0;
    try {
        if (mem_.uploads_in_flight > 0) {  // tensors still being filled by dx_exec_upload_async: this op waits for those it names
            auto wait = [&](const Param &q) {
                if ((q.dtype.category & (CAT_TENSOR | CAT_LISTTENSOR)) == 0) return;
                std::string names = q.textvalue;
                trim_chars(names, "[]");
                std::istringstream ns(names);
                std::string nm;
                while (ns >> nm)
                    if (mem_.exists_tensor(nm)) {
                        Tensor &t = *mem_.get_tensor(nm);
                        if (t.upload_in_flight) {
                            mem_.wait_ready(t);
                            --mem_.uploads_in_flight;
                        }
                    }
            };
            for (const auto &q : tf->args) wait(q);
            for (const auto &q : tf->returns) wait(q);
        }
        if (mem_.shard.comm && dx_comm_pending(mem_.shard.comm, nullptr)) {
            // A cross-rank reduction left its combine for later.  Compute ops that do not touch its output go ahead
            // (they are what hides the skew between the ranks); anything that reads or writes that tensor, and every
            // op that is not plain compute (lifetime, io, args), waits for it.
            static const char *compute[] = {"elementwise", "reduce", "changeshape", "matmul", "fused", "init"};
            bool plain = false;
            for (const char *c : compute) plain = plain || tf->tftype == c;
            bool touches = !plain;
            auto look = [&](const Param &q) {
                if (touches || (q.dtype.category & (CAT_TENSOR | CAT_LISTTENSOR)) == 0) return;
                std::string names = q.textvalue;
                trim_chars(names, "[]");
                std::istringstream ns(names);
                std::string nm;
                while (ns >> nm)
                    if (mem_.exists_tensor(nm)) {
                        const TensorPtr t = mem_.get_tensor(nm);
                        touches = touches || mem_.comm_pending_in(t->data, size_t(std::max<int64_t>(t->shape.bytes(), 0)));
                    }
            };
            for (const auto &q : tf->args) look(q);
            for (const auto &q : tf->returns) look(q);
            if (touches) mem_.flush_comm();
        }
        const int repeat = tf->metadata.benchmark_repeat > 1 ? tf->metadata.benchmark_repeat : 1;
        for (int i = 0; i < repeat && rc == 0; ++i) rc = tf->run(mem_, message);
        // a timed request wants the device to have finished before finish_at is taken
        if (tf->metadata.benchmark_repeat > 0) {
            mem_.flush_comm();
            cudaStreamSynchronize(static_cast<cudaStream_t>(mem_.stream()));
        }
    } catch (const std::exception &e) {
        rc = 1;
        message = e.what();
    } catch (...) {
        rc = 1;
        message = "unknown exception";
    }
    ++ops_run_;
    if (rc != 0) resp.error(message);
    else resp.finish("");
    return resp;
}

void Executor::set_shard(int rank, int world, size_t min_bytes, dx_comm *comm) {
    if (world < 1 || rank < 0 || rank >= world) throw std::invalid_argument("set_shard: rank " + std::to_string(rank) + " of " + std::to_string(world));
    if (world > 1 && !comm) throw std::invalid_argument("set_shard: more than one rank needs a connected communicator");
    if (comm && (dx_comm_rank(comm) != rank || dx_comm_world(comm) != world)) throw std::invalid_argument("set_shard: the communicator was created for another rank or world size");
    std::lock_guard<std::mutex> lk(mu_);
    mem_.shard.rank = rank;
    mem_.shard.world = world;
    mem_.shard.min_bytes = min_bytes;
    mem_.shard.comm = world > 1 ? comm : nullptr;
}

OpResp Executor::run_line(const std::string &ir) {
    TF call;
    call.metadata.recv_at = std::chrono::system_clock::now();
    try {
        call.parse(ir);
    } catch (const std::exception &e) {
        OpResp resp;
        resp.recv_at = call.metadata.recv_at;
        resp.start_at = resp.recv_at;
        resp.error(e.what());
        return resp;
    }
    return run(call);
}

std::vector<OpResp> Executor::run_program(const std::string &text) {
    std::vector<std::string> lines;
    {
        std::istringstream ss(text);
        std::string line;
        while (std::getline(ss, line)) {
            if (!line.empty() && line.back() == '\r') line.pop_back();
            if (line.find_first_not_of(" \t") != std::string::npos) lines.push_back(line);
        }
    }
    std::vector<OpResp> replies;
    replies.reserve(lines.size());
    const auto now = std::chrono::system_clock::now();
    std::vector<TF> program(lines.size());
    bool parsed = fuse && lines.size() > 1;
    for (size_t i = 0; parsed && i < lines.size(); ++i) {
        try {
            program[i].metadata.recv_at = now;
            program[i].parse(lines[i]);
        } catch (const std::exception &) {
            parsed = false;  // the line-by-line path reports the error where it belongs
        }
    }
    if (!parsed) {
        for (const auto &l : lines) replies.push_back(run_line(l));
        return replies;
    }
    const std::vector<PlanItem> plan = plan_fusion(program, mem_, &fusion_);
    for (size_t i = 0; i < program.size(); ++i) {
        if (plan[i].kind == PlanItem::ABSORBED) {
            OpResp r;
            r.id = program[i].metadata.id;
            r.recv_at = now;
            r.start_at = std::chrono::system_clock::now();
            r.finish("");
            replies.push_back(r);
        } else {
            replies.push_back(run(plan[i].kind == PlanItem::FUSED ? plan[i].fused : program[i]));
        }
    }
    return replies;
}

CompiledProgram::~CompiledProgram() {
    if (exec) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(exec));
    if (graph) cudaGraphDestroy(static_cast<cudaGraph_t>(graph));
}

std::shared_ptr<CompiledProgram> Executor::compile(const std::string &text, std::string *error) {
    auto failed = [&](const std::string &why) {
        if (error) *error = why;
        return std::shared_ptr<CompiledProgram>();
    };
    std::vector<TF> program;
    {
        std::istringstream ss(text);
        std::string line;
        while (std::getline(ss, line)) {
            if (!line.empty() && line.back() == '\r') line.pop_back();
            if (line.find_first_not_of(" \t") == std::string::npos) continue;
            try {
                program.emplace_back(line);
            } catch (const std::exception &e) {
                return failed("line " + std::to_string(program.size() + 1) + ": " + e.what());
            }
        }
    }
    if (program.empty()) return failed("empty program");
    FusionStats before = fusion_;
    const std::vector<PlanItem> plan = fuse ? plan_fusion(program, mem_, &fusion_) : std::vector<PlanItem>(program.size());
    std::vector<TF> ops;
    static const char *refused[] = {"newtensor", "deltensor", "renametensor", "print", "save", "load", "loadtensordata", "argset", "vecset"};
    for (size_t i = 0; i < program.size(); ++i) {
        if (plan[i].kind == PlanItem::ABSORBED) continue;
        const TF &t = plan[i].kind == PlanItem::FUSED ? plan[i].fused : program[i];
        for (const char *r : refused)
            if (t.name == r) return failed("line " + std::to_string(i + 1) + ": " + t.name + " cannot be part of a compiled program (compute ops only)");
        if (t.metadata.benchmark_repeat > 0) return failed("line " + std::to_string(i + 1) + ": a timed line (benchmark.repeat) cannot be captured");
        ops.push_back(t);
    }
    if (ops.empty()) return failed("nothing to run after fusion");
    // pass 1: a normal run — grows the workspace, does first-call set-up, and its results stand
    for (size_t i = 0; i < ops.size(); ++i) {
        const OpResp r = run(ops[i]);
        if (r.result != "ok") return failed(ops[i].name + ": " + r.message);
    }
    cudaStream_t st = static_cast<cudaStream_t>(mem_.stream());
    cudaSetDevice(mem_.device());
    try {
        mem_.flush_comm();
    } catch (const std::exception &e) {
        return failed(e.what());
    }
    if (cudaStreamSynchronize(st) != cudaSuccess) return failed(std::string("stream: ") + cudaGetErrorString(cudaGetLastError()));
    // pass 2: the same ops, captured instead of executed
    auto out = std::make_shared<CompiledProgram>();
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
        return failed(std::string("cudaStreamBeginCapture: ") + cudaGetErrorString(cudaGetLastError()));
    mem_.capturing = true;
    std::string why;
    for (size_t i = 0; i < ops.size() && why.empty(); ++i) {
        const OpResp r = run(ops[i]);
        if (r.result != "ok") why = ops[i].name + ": " + r.message;
    }
    if (why.empty()) {
        try {
            mem_.flush_comm();  // a combine left open by the last cross-rank reduction belongs to the program
        } catch (const std::exception &e) {
            why = e.what();
        }
    }
    mem_.capturing = false;
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(st, &graph);
    if (why.empty() && ce != cudaSuccess) why = std::string("cudaStreamEndCapture: ") + cudaGetErrorString(ce);
    if (!why.empty()) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return failed(why);
    }
    out->graph = graph;
    cudaGraphExec_t exec = nullptr;
    if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) return failed(std::string("cudaGraphInstantiate: ") + cudaGetErrorString(cudaGetLastError()));
    out->exec = exec;
    size_t nodes = 0;
    cudaGraphGetNodes(graph, nullptr, &nodes);
    out->nodes = nodes;
    out->lines = program.size();
    out->ops = ops.size();
    out->fused_groups = size_t((fusion_.rmsnorm_groups - before.rmsnorm_groups) + (fusion_.softmax_groups - before.softmax_groups));
    out->scratch_generation = mem_.scratch_generation();
    for (const TF &t : ops) {
        auto note = [&](const Param &q) {
            if ((q.dtype.category & (CAT_TENSOR | CAT_LISTTENSOR)) == 0) return;
            std::string names = q.textvalue;
            trim_chars(names, "[]");
            std::istringstream ns(names);
            std::string nm;
            while (ns >> nm) {
                if (!mem_.exists_tensor(nm)) continue;
                bool seen = false;
                for (const auto &r : out->refs) seen |= (r.name == nm);
                if (seen) continue;
                const TensorPtr p = mem_.get_tensor(nm);
                out->refs.push_back({nm, p->data, p->shape.dtype, p->shape.shape});
            }
        };
        for (const auto &q : t.args) note(q);
        for (const auto &q : t.returns) note(q);
    }
    return out;
}

int Executor::replay(CompiledProgram &program, std::string *error) {
    auto failed = [&](const std::string &why) {
        if (error) *error = why;
        return 1;
    };
    if (!program.exec) return failed("program was not compiled");
    std::lock_guard<std::mutex> lk(mu_);
    if (program.scratch_generation != mem_.scratch_generation())
        return failed("stale program: the reduce workspace moved since it was compiled; compile it again");
    for (const auto &r : program.refs) {
        if (!mem_.exists_tensor(r.name)) return failed("stale program: tensor " + r.name + " no longer exists; compile it again");
        const TensorPtr p = mem_.get_tensor(r.name);
        if (p->data != r.data || p->shape.dtype != r.precision || p->shape.shape != r.shape)
            return failed("stale program: tensor " + r.name + " changed storage, dtype or shape; compile it again");
        if (p->upload_in_flight) {  // an asynchronous upload into a tensor the program uses: the graph launch waits for it
            mem_.wait_ready(*p);
            --mem_.uploads_in_flight;
        }
    }
    try {
        mem_.flush_comm();
    } catch (const std::exception &e) {
        return failed(e.what());
    }
    cudaSetDevice(mem_.device());
    const cudaError_t e = cudaGraphLaunch(static_cast<cudaGraphExec_t>(program.exec), static_cast<cudaStream_t>(mem_.stream()));
    if (e != cudaSuccess) return failed(std::string("cudaGraphLaunch: ") + cudaGetErrorString(e));
    ops_run_ += program.ops;
    return 0;
}

}  // namespace dxh
