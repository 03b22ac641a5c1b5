// GGUF reader of the Q8_0 path (host only): header, metadata, tensor table, bounded reads.
// Interface and the reference code it stands in for: include/aotx_gguf_b200.h.
//
// The file is mapped read-only and the header is parsed by a bounds-checked cursor over the
// mapping; scalar and string metadata and the tensor table (with an index by name) are kept,
// array values stay in the file until a getter asks for one.  Tensor bytes are read with pread on the descriptor, so a read of a file
// that was cut short after open fails with a code instead of a fault on a mapped page.
//
// The structural checks are the ones the reference's reader makes (disk/modelfile/gguf.c,
// disk/modelfile/meta.c), so that both readers accept and refuse the same files: version 3,
// counts that the file could hold, keys under 256 bytes and names under 128 bytes without zero
// bytes, known value types, booleans 0 or 1, no nested arrays, arrays of at most 8 Mi elements,
// 1 to 4 non-zero dimensions, quantised rows a whole number of blocks, alignment a power of two
// up to 65536, tensors on the alignment and inside the tensor bytes, unique keys and names, and
// a head (everything before the tensor bytes) of at most 256 MiB.  The reference also bounds
// the memory its own parser allocates (512 MiB, mostly copies of string arrays); this reader
// copies an array only when it is asked for and has no such bound.
#include "../../include/aotx_gguf_b200.h"

#include <errno.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

constexpr uint64_t kHeadLimit = 256ull * 1024ull * 1024ull;
constexpr uint64_t kPairLeast = 12;
constexpr uint64_t kTensorLeast = 24;
constexpr uint64_t kKeyBytes = 256;
constexpr uint64_t kArrayLimit = 8ull * 1024ull * 1024ull;
constexpr uint32_t kMagic = 0x46554747u; // "GGUF"
constexpr uint32_t kVersion = 3;

enum ValueType : uint32_t {
    kU8 = 0, kI8, kU16, kI16, kU32, kI32, kF32, kBool, kString, kArray, kU64, kI64, kF64
};

struct BlockLayout {
    uint32_t type;
    uint32_t weights;
    uint32_t bytes;
};

// Block types with a known layout: weights per block, bytes per block
// (disk/modelfile/modelfile.h:58-88).
const BlockLayout kLayouts[] = {
    {0, 1, 4},      // F32
    {1, 1, 2},      // F16
    {2, 32, 18},    // Q4_0
    {3, 32, 20},    // Q4_1
    {6, 32, 22},    // Q5_0
    {7, 32, 24},    // Q5_1
    {8, 32, 34},    // Q8_0
    {10, 256, 84},  // Q2_K
    {11, 256, 110}, // Q3_K
    {12, 256, 144}, // Q4_K
    {13, 256, 176}, // Q5_K
    {14, 256, 210}, // Q6_K
};

const BlockLayout *layout_of(uint32_t type)
{
    for (const BlockLayout &l : kLayouts) {
        if (l.type == type) {
            return &l;
        }
    }
    return nullptr;
}

unsigned width_of(uint32_t type)
{
    switch (type) {
    case kU8: case kI8: case kBool: return 1;
    case kU16: case kI16: return 2;
    case kU32: case kI32: case kF32: return 4;
    case kU64: case kI64: case kF64: return 8;
    default: return 0;
    }
}

bool is_signed(uint32_t type)
{
    return type == kI8 || type == kI16 || type == kI32 || type == kI64;
}

struct Meta {
    uint32_t type = 0;
    uint32_t element_type = 0;
    uint64_t count = 0;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0.0;
    std::string text;
    // An array's elements stay in the file; `array_pos` is the file offset of the first one and
    // `array_bytes` their span.  A getter reads and converts them the first time it is asked.
    uint64_t array_pos = 0;
    uint64_t array_bytes = 0;
    mutable bool loaded = false;
    mutable bool fits = false;            // every element fits the type the getter gives
    mutable std::vector<int32_t> i32;
    mutable std::vector<float> f32;
    mutable std::vector<uint8_t> run;      // booleans, or the bytes of all strings
    mutable std::vector<uint64_t> offsets; // count + 1 entries into `run`
};

} // namespace

struct aotx_gguf {
    int fd = -1;
    std::string path;
    uint64_t file_bytes = 0;
    uint64_t header_bytes = 0;
    uint64_t data_offset = 0;
    uint64_t data_bytes = 0;
    uint32_t alignment = 32;
    std::unordered_map<std::string, Meta> meta;
    std::vector<aotx_gguf_tensor_info> tensors;
    std::unordered_map<std::string, size_t> by_name;
};

namespace {

// The parse: a cursor over the mapped file.  `fail` records the first reason and every later
// step becomes a no-op, so the grammar below reads straight through.
class Parse {
public:
    Parse(aotx_gguf *file, const unsigned char *base) : file_(file), base_(base) {}

    bool ok() const { return reason_ == nullptr; }
    const char *reason() const { return reason_; }
    uint64_t pos() const { return pos_; }

    void fail(const char *reason)
    {
        if (reason_ == nullptr) {
            reason_ = reason;
        }
    }

    const unsigned char *take(uint64_t bytes)
    {
        if (!ok()) {
            return nullptr;
        }
        if (bytes > file_->file_bytes || pos_ > file_->file_bytes - bytes) {
            fail("a field goes past the end of the file");
            return nullptr;
        }
        if (pos_ + bytes > kHeadLimit) {
            fail("the head of the file is too long");
            return nullptr;
        }
        const unsigned char *at = base_ + pos_;
        pos_ += bytes;
        return at;
    }

    uint64_t number(unsigned width)
    {
        const unsigned char *at = take(width);
        uint64_t value = 0;
        if (at != nullptr) {
            for (unsigned i = 0; i < width; ++i) {
                value |= (uint64_t)at[i] << (8u * i);
            }
        }
        return value;
    }

    // length-prefixed bytes; the view stays valid while the mapping does
    const unsigned char *text(uint64_t *length)
    {
        uint64_t len = number(8);
        const unsigned char *at = take(len);
        *length = at != nullptr ? len : 0;
        return at;
    }

    void header(uint64_t *tensor_count, uint64_t *meta_count)
    {
        if (number(4) != kMagic && ok()) {
            fail("the first four bytes are not GGUF");
        }
        if (number(4) != kVersion && ok()) {
            fail("the version is not 3");
        }
        *tensor_count = number(8);
        *meta_count = number(8);
        if (!ok()) {
            return;
        }
        if (*tensor_count > kHeadLimit / kTensorLeast || *meta_count > kHeadLimit / kPairLeast) {
            fail("the field counts exceed the header limit");
        } else if (*tensor_count > file_->file_bytes / kTensorLeast) {
            fail("the tensor count is larger than the file can hold");
        } else if (*meta_count > file_->file_bytes / kPairLeast) {
            fail("the metadata count is larger than the file can hold");
        }
    }

    void scalar(Meta &m, uint32_t type)
    {
        unsigned width = width_of(type);
        if (width == 0) {
            fail("a metadata value has a type that is not known");
            return;
        }
        uint64_t raw = number(width);
        m.u = raw;
        if (is_signed(type) && width < 8 && (raw >> (8u * width - 1u)) != 0) {
            m.i = (int64_t)(raw | ~((1ull << (8u * width)) - 1ull));
        } else {
            m.i = (int64_t)raw;
        }
        if (type == kF32) {
            float v;
            uint32_t bits = (uint32_t)raw;
            std::memcpy(&v, &bits, sizeof v);
            m.f = (double)v;
        } else if (type == kF64) {
            std::memcpy(&m.f, &raw, sizeof m.f);
        }
        if (type == kBool && raw > 1u) {
            fail("a boolean value is not 0 or 1");
        }
    }

    void array(Meta &m)
    {
        m.element_type = (uint32_t)number(4);
        m.count = number(8);
        if (!ok()) {
            return;
        }
        if (m.element_type == kArray) {
            fail("an array holds an array, which the format does not allow");
            return;
        }
        if (m.count > kArrayLimit) {
            fail("an array holds more elements than the limit");
            return;
        }
        m.array_pos = pos_;
        if (m.element_type == kString) {
            if (m.count > (file_->file_bytes - pos_) / 8u || pos_ > kHeadLimit
                || m.count > (kHeadLimit - pos_) / 8u) {
                fail("a string array count exceeds the remaining header");
                return;
            }
            for (uint64_t i = 0; i < m.count && ok(); ++i) {
                uint64_t length = 0;
                text(&length);
            }
            m.array_bytes = pos_ - m.array_pos;
            return;
        }
        unsigned width = width_of(m.element_type);
        if (width == 0) {
            fail("an array holds a type that is not known");
            return;
        }
        const unsigned char *at = take(m.count * width);
        m.array_bytes = m.count * width;
        if (at != nullptr && m.element_type == kBool) {
            for (uint64_t i = 0; i < m.count; ++i) {
                if (at[i] > 1u) {
                    fail("a boolean array value is not 0 or 1");
                    return;
                }
            }
        }
    }

    void metadata(uint64_t count)
    {
        // counts come from the file: reserve for a plausible table, grow for the rest
        file_->meta.reserve((size_t)(count < 4096 ? count : 4096));
        for (uint64_t i = 0; i < count && ok(); ++i) {
            uint64_t key_bytes = 0;
            const unsigned char *key = text(&key_bytes);
            if (!ok()) {
                return;
            }
            if (key_bytes >= kKeyBytes) {
                fail("a metadata key is too long");
                return;
            }
            if (key_bytes != 0 && std::memchr(key, 0, (size_t)key_bytes) != nullptr) {
                fail("a metadata key holds a zero byte");
                return;
            }
            Meta m;
            m.type = (uint32_t)number(4);
            if (!ok()) {
                return;
            }
            if (m.type == kArray) {
                array(m);
            } else if (m.type == kString) {
                uint64_t length = 0;
                const unsigned char *bytes = text(&length);
                if (bytes != nullptr) {
                    m.text.assign(reinterpret_cast<const char *>(bytes), (size_t)length);
                }
            } else {
                scalar(m, m.type);
            }
            if (!ok()) {
                return;
            }
            std::string name(reinterpret_cast<const char *>(key), (size_t)key_bytes);
            if (!file_->meta.emplace(std::move(name), std::move(m)).second) {
                repeated_key_ = true; // reported after the tensor table, as the reference orders it
            }
        }
    }

    void tensor(aotx_gguf_tensor_info &t)
    {
        uint64_t name_bytes = 0;
        const unsigned char *name = text(&name_bytes);
        if (!ok()) {
            return;
        }
        if (name_bytes >= AOTX_GGUF_NAME_BYTES) {
            fail("a tensor name is too long");
            return;
        }
        if (name_bytes == 0 || std::memchr(name, 0, (size_t)name_bytes) != nullptr) {
            fail("a tensor name is empty or holds a zero byte");
            return;
        }
        std::memset(&t, 0, sizeof t);
        std::memcpy(t.name, name, (size_t)name_bytes);
        uint64_t dims = number(4);
        if (!ok()) {
            return;
        }
        if (dims == 0 || dims > AOTX_GGUF_DIMS) {
            fail("a tensor has a dimension count that is not 1 to 4");
            return;
        }
        t.dim_count = (uint32_t)dims;
        for (uint32_t d = 0; d < AOTX_GGUF_DIMS; ++d) {
            t.dims[d] = d < t.dim_count ? number(8) : 1;
        }
        t.type = (uint32_t)number(4);
        t.offset = number(8);
        if (!ok()) {
            return;
        }
        uint64_t weights = 1;
        for (uint32_t d = 0; d < t.dim_count; ++d) {
            if (t.dims[d] == 0) {
                fail("a tensor dimension is zero");
                return;
            }
            if (weights > UINT64_MAX / t.dims[d]) {
                fail("the weight count of a tensor is too large");
                return;
            }
            weights *= t.dims[d];
        }
        const BlockLayout *layout = layout_of(t.type);
        if (layout == nullptr) {
            t.bytes = 0; // no layout known here: the entry stays in the table, nothing streams
            return;
        }
        if (layout->weights > 1 && (t.dims[0] % layout->weights) != 0) {
            fail("a quantized row is not a whole count of blocks");
            return;
        }
        if (weights / layout->weights > UINT64_MAX / layout->bytes) {
            fail("the byte count of a tensor is too large");
            return;
        }
        t.bytes = weights / layout->weights * layout->bytes;
    }

    void table(uint64_t count)
    {
        file_->tensors.reserve((size_t)(count < 4096 ? count : 4096));
        for (uint64_t i = 0; i < count && ok(); ++i) {
            aotx_gguf_tensor_info t;
            tensor(t);
            if (ok()) {
                file_->tensors.push_back(t);
            }
        }
        if (!ok()) {
            return;
        }
        uint64_t align = 32;
        auto found = file_->meta.find("general.alignment");
        if (found != file_->meta.end()) {
            const Meta &m = found->second;
            bool whole = width_of(m.type) != 0 && m.type != kF32 && m.type != kF64;
            bool fits = whole && !(is_signed(m.type) && m.i < 0)
                     && (is_signed(m.type) ? (uint64_t)m.i : m.u) <= 0xffffffffull;
            if (!fits) {
                fail("the alignment key holds another type");
                return;
            }
            align = is_signed(m.type) ? (uint64_t)m.i : m.u;
        }
        if (align == 0 || align > 65536u || (align & (align - 1u)) != 0) {
            fail("the alignment is not a power of two from 1 to 65536");
            return;
        }
        file_->alignment = (uint32_t)align;
        file_->header_bytes = pos_;
        uint64_t pad = (pos_ % align) == 0 ? 0 : align - (pos_ % align);
        if (pad > file_->file_bytes - pos_) {
            fail("the tensor bytes start past the end of the file");
            return;
        }
        file_->data_offset = pos_ + pad;
        file_->data_bytes = file_->file_bytes - file_->data_offset;
        for (const aotx_gguf_tensor_info &t : file_->tensors) {
            if ((t.offset % align) != 0) {
                fail("a tensor offset is not on the alignment");
                return;
            }
            if (t.bytes > file_->data_bytes || t.offset > file_->data_bytes - t.bytes) {
                fail("a tensor goes past the end of the tensor bytes");
                return;
            }
        }
        if (repeated_key_) {
            fail("a metadata key is repeated");
            return;
        }
        file_->by_name.reserve(file_->tensors.size());
        for (size_t i = 0; i < file_->tensors.size(); ++i) {
            if (!file_->by_name.emplace(file_->tensors[i].name, i).second) {
                fail("a tensor name is repeated");
                return;
            }
        }
    }

private:
    aotx_gguf *file_;
    const unsigned char *base_;
    uint64_t pos_ = 0;
    const char *reason_ = nullptr;
    bool repeated_key_ = false;
};

const Meta *find_meta(const aotx_gguf *file, const char *key)
{
    if (file == nullptr || key == nullptr) {
        return nullptr;
    }
    auto found = file->meta.find(key);
    return found == file->meta.end() ? nullptr : &found->second;
}

// any whole-number type that is not negative
int whole_value(const Meta &m, uint64_t *out)
{
    if (width_of(m.type) == 0 || m.type == kF32 || m.type == kF64) {
        return 2;
    }
    if (is_signed(m.type)) {
        if (m.i < 0) {
            return 2;
        }
        *out = (uint64_t)m.i;
        return 0;
    }
    *out = m.u;
    return 0;
}

} // namespace

extern "C" int aotx_gguf_open(const char *path, aotx_gguf **out)
{
    if (path == nullptr || out == nullptr) {
        return AOTX_GGUF_ERR_READ;
    }
    *out = nullptr;
    aotx_gguf *file = new (std::nothrow) aotx_gguf();
    if (file == nullptr) {
        return AOTX_GGUF_ERR_READ;
    }
    file->path = path;
    file->fd = open(path, O_RDONLY | O_NONBLOCK | O_CLOEXEC);
    struct stat st;
    if (file->fd < 0 || fstat(file->fd, &st) != 0 || !S_ISREG(st.st_mode)) {
        std::fprintf(stderr, "aotx_gguf: %s: not a regular file that opens\n", path);
        aotx_gguf_close(file);
        return AOTX_GGUF_ERR_READ;
    }
    file->file_bytes = (uint64_t)st.st_size;
    // Only the head is parsed; the mapping covers at most the head limit.
    const uint64_t map_bytes = file->file_bytes < kHeadLimit ? file->file_bytes : kHeadLimit;
    void *map = nullptr;
    if (map_bytes > 0) {
        map = mmap(nullptr, (size_t)map_bytes, PROT_READ, MAP_PRIVATE, file->fd, 0);
        if (map == MAP_FAILED) {
            std::fprintf(stderr, "aotx_gguf: %s: the file does not map\n", path);
            aotx_gguf_close(file);
            return AOTX_GGUF_ERR_READ;
        }
    }
    Parse parse(file, static_cast<const unsigned char *>(map));
    uint64_t tensor_count = 0, meta_count = 0;
    bool memory = true;
    try {
        parse.header(&tensor_count, &meta_count);
        if (parse.ok()) {
            parse.metadata(meta_count);
        }
        if (parse.ok()) {
            parse.table(tensor_count);
        }
    } catch (const std::bad_alloc &) {
        memory = false;
    }
    if (map != nullptr) {
        munmap(map, (size_t)map_bytes);
    }
    if (!memory || !parse.ok()) {
        std::fprintf(stderr, "aotx_gguf: %s: %s\n", path,
                     memory ? parse.reason() : "the memory for the tables is not there");
        aotx_gguf_close(file);
        return AOTX_GGUF_ERR_FORMAT;
    }
    *out = file;
    return AOTX_GGUF_OK;
}

extern "C" void aotx_gguf_close(aotx_gguf *file)
{
    if (file == nullptr) {
        return;
    }
    if (file->fd >= 0) {
        close(file->fd);
    }
    delete file;
}

extern "C" uint64_t aotx_gguf_file_bytes(const aotx_gguf *file)
{
    return file != nullptr ? file->file_bytes : 0;
}

extern "C" uint64_t aotx_gguf_header_bytes(const aotx_gguf *file)
{
    return file != nullptr ? file->header_bytes : 0;
}

extern "C" uint64_t aotx_gguf_data_bytes(const aotx_gguf *file)
{
    return file != nullptr ? file->data_bytes : 0;
}

extern "C" uint32_t aotx_gguf_alignment(const aotx_gguf *file)
{
    return file != nullptr ? file->alignment : 0;
}

extern "C" uint64_t aotx_gguf_tensor_count(const aotx_gguf *file)
{
    return file != nullptr ? file->tensors.size() : 0;
}

extern "C" int aotx_gguf_tensor(const aotx_gguf *file, uint64_t index, aotx_gguf_tensor_info *info)
{
    if (file == nullptr || info == nullptr || index >= file->tensors.size()) {
        return 1;
    }
    *info = file->tensors[(size_t)index];
    return 0;
}

extern "C" int aotx_gguf_find(const aotx_gguf *file, const char *name, aotx_gguf_tensor_info *info)
{
    if (file == nullptr || name == nullptr || info == nullptr) {
        return 1;
    }
    auto found = file->by_name.find(name);
    if (found == file->by_name.end()) {
        return 1;
    }
    *info = file->tensors[found->second];
    return 0;
}

extern "C" int aotx_gguf_u64(const aotx_gguf *file, const char *key, uint64_t *value)
{
    const Meta *m = find_meta(file, key);
    if (m == nullptr || value == nullptr) {
        return 1;
    }
    return whole_value(*m, value);
}

extern "C" int aotx_gguf_u32(const aotx_gguf *file, const char *key, uint32_t *value)
{
    const Meta *m = find_meta(file, key);
    if (m == nullptr || value == nullptr) {
        return 1;
    }
    uint64_t wide = 0;
    int rc = whole_value(*m, &wide);
    if (rc != 0) {
        return rc;
    }
    if (wide > 0xffffffffull) {
        return 2;
    }
    *value = (uint32_t)wide;
    return 0;
}

extern "C" int aotx_gguf_f32(const aotx_gguf *file, const char *key, float *value)
{
    const Meta *m = find_meta(file, key);
    if (m == nullptr || value == nullptr) {
        return 1;
    }
    if (m->type != kF32 && m->type != kF64) {
        return 2;
    }
    *value = (float)m->f;
    return 0;
}

extern "C" int aotx_gguf_string(const aotx_gguf *file, const char *key, const char **value, size_t *length)
{
    const Meta *m = find_meta(file, key);
    if (m == nullptr || value == nullptr) {
        return 1;
    }
    if (m->type != kString) {
        return 2;
    }
    *value = m->text.c_str();
    if (length != nullptr) {
        *length = m->text.size();
    }
    return 0;
}

extern "C" int aotx_gguf_array(const aotx_gguf *file, const char *key, uint32_t *element_type, uint64_t *count)
{
    const Meta *m = find_meta(file, key);
    if (m == nullptr) {
        return 1;
    }
    if (m->type != kArray) {
        return 2;
    }
    if (element_type != nullptr) {
        *element_type = m->element_type;
    }
    if (count != nullptr) {
        *count = m->count;
    }
    return 0;
}

namespace {

bool read_at(const aotx_gguf *file, uint64_t from, uint64_t bytes, unsigned char *out)
{
    while (bytes > 0) {
        ssize_t got = pread(file->fd, out, (size_t)bytes, (off_t)from);
        if (got < 0 && errno == EINTR) {
            continue;
        }
        if (got <= 0) {
            return false;
        }
        out += got;
        from += (uint64_t)got;
        bytes -= (uint64_t)got;
    }
    return true;
}

uint64_t little(const unsigned char *at, unsigned width)
{
    uint64_t value = 0;
    for (unsigned i = 0; i < width; ++i) {
        value |= (uint64_t)at[i] << (8u * i);
    }
    return value;
}

// Bring the elements of an array value in from the file, once, in the form its getter gives.
// The structure was checked at open, so the bytes parse.
bool load_array(const aotx_gguf *file, const Meta &m)
{
    if (m.loaded) {
        return true;
    }
    std::vector<unsigned char> raw((size_t)m.array_bytes);
    if (!raw.empty() && !read_at(file, m.array_pos, m.array_bytes, raw.data())) {
        return false;
    }
    if (m.element_type == kString) {
        m.offsets.assign((size_t)m.count + 1, 0);
        uint64_t at = 0;
        for (uint64_t i = 0; i < m.count; ++i) {
            const uint64_t length = little(raw.data() + at, 8);
            at += 8;
            m.run.insert(m.run.end(), raw.begin() + (ptrdiff_t)at, raw.begin() + (ptrdiff_t)(at + length));
            at += length;
            m.offsets[(size_t)i + 1] = m.run.size();
        }
        m.fits = true;
    } else if (m.element_type == kI32 || m.element_type == kU32) {
        m.i32.assign((size_t)m.count, 0);
        m.fits = true;
        for (uint64_t i = 0; i < m.count; ++i) {
            const uint64_t bits = little(raw.data() + 4 * i, 4);
            if (m.element_type == kU32 && bits > 0x7fffffffull) {
                m.fits = false; // the getter gives int32; the reference withholds such an array too
            }
            m.i32[(size_t)i] = (int32_t)(uint32_t)bits;
        }
    } else if (m.element_type == kF32) {
        m.f32.assign((size_t)m.count, 0.0f);
        for (uint64_t i = 0; i < m.count; ++i) {
            const uint32_t bits = (uint32_t)little(raw.data() + 4 * i, 4);
            std::memcpy(&m.f32[(size_t)i], &bits, 4);
        }
        m.fits = true;
    } else if (m.element_type == kBool) {
        m.run.assign(raw.begin(), raw.end());
        m.fits = true;
    }
    m.loaded = true;
    return true;
}

const Meta *find_array(const aotx_gguf *file, const char *key, int *code)
{
    const Meta *m = find_meta(file, key);
    if (m == nullptr) {
        *code = 1;
        return nullptr;
    }
    if (m->type != kArray) {
        *code = 2;
        return nullptr;
    }
    *code = 0;
    return m;
}

// a pointer that is never null, also for an empty array
template <typename T>
const T *data_or_spot(const std::vector<T> &values)
{
    static const T spot = T();
    return values.empty() ? &spot : values.data();
}

} // namespace

extern "C" int aotx_gguf_i32s(const aotx_gguf *file, const char *key, const int32_t **values, uint64_t *count)
{
    int code = 0;
    const Meta *m = values != nullptr ? find_array(file, key, &code) : nullptr;
    if (values == nullptr) {
        return 1;
    }
    if (m == nullptr) {
        return code;
    }
    if ((m->element_type != kI32 && m->element_type != kU32) || !load_array(file, *m) || !m->fits) {
        return 2;
    }
    *values = data_or_spot(m->i32);
    if (count != nullptr) {
        *count = m->count;
    }
    return 0;
}

extern "C" int aotx_gguf_f32s(const aotx_gguf *file, const char *key, const float **values, uint64_t *count)
{
    int code = 0;
    const Meta *m = values != nullptr ? find_array(file, key, &code) : nullptr;
    if (values == nullptr) {
        return 1;
    }
    if (m == nullptr) {
        return code;
    }
    if (m->element_type != kF32 || !load_array(file, *m)) {
        return 2;
    }
    *values = data_or_spot(m->f32);
    if (count != nullptr) {
        *count = m->count;
    }
    return 0;
}

extern "C" int aotx_gguf_bools(const aotx_gguf *file, const char *key, const uint8_t **values, uint64_t *count)
{
    int code = 0;
    const Meta *m = values != nullptr ? find_array(file, key, &code) : nullptr;
    if (values == nullptr) {
        return 1;
    }
    if (m == nullptr) {
        return code;
    }
    if (m->element_type != kBool || !load_array(file, *m)) {
        return 2;
    }
    *values = data_or_spot(m->run);
    if (count != nullptr) {
        *count = m->count;
    }
    return 0;
}

extern "C" int aotx_gguf_strings(const aotx_gguf *file, const char *key, aotx_gguf_string_array *array)
{
    int code = 0;
    const Meta *m = array != nullptr ? find_array(file, key, &code) : nullptr;
    if (array == nullptr) {
        return 1;
    }
    if (m == nullptr) {
        return code;
    }
    if (m->element_type != kString || !load_array(file, *m)) {
        return 2;
    }
    array->count = m->count;
    array->bytes = data_or_spot(m->run);
    array->offsets = m->offsets.data();
    return 0;
}

extern "C" int aotx_gguf_read(const aotx_gguf *file, uint64_t offset, uint64_t bytes, void *buffer)
{
    if (file == nullptr || (buffer == nullptr && bytes > 0)) {
        return AOTX_GGUF_ERR_READ;
    }
    if (bytes > file->data_bytes || offset > file->data_bytes - bytes) {
        std::fprintf(stderr, "aotx_gguf: %s: a read goes past the end of the tensor bytes\n",
                     file->path.c_str());
        return AOTX_GGUF_ERR_FORMAT;
    }
    unsigned char *at = static_cast<unsigned char *>(buffer);
    uint64_t from = file->data_offset + offset;
    uint64_t left = bytes;
    while (left > 0) {
        // one call moves at most 2 GiB less a page on Linux; short counts are normal
        size_t want = left < (1ull << 30) ? (size_t)left : (size_t)(1ull << 30);
        ssize_t got = pread(file->fd, at, want, (off_t)from);
        if (got < 0 && errno == EINTR) {
            continue;
        }
        if (got <= 0) {
            std::fprintf(stderr, "aotx_gguf: %s: a tensor read %s\n", file->path.c_str(),
                         got == 0 ? "found the end of the file" : "failed");
            return AOTX_GGUF_ERR_READ;
        }
        at += got;
        from += (uint64_t)got;
        left -= (uint64_t)got;
    }
    return AOTX_GGUF_OK;
}

extern "C" int aotx_gguf_read_threads(const aotx_gguf *file, uint64_t offset, uint64_t bytes, void *buffer,
                                      uint32_t threads)
{
    const uint64_t slice_least = 4ull * 1024ull * 1024ull; // below this a second thread does not pay
    uint64_t slices = bytes / slice_least;
    if (slices > threads) {
        slices = threads;
    }
    if (slices <= 1 || file == nullptr || buffer == nullptr) {
        return aotx_gguf_read(file, offset, bytes, buffer);
    }
    if (bytes > file->data_bytes || offset > file->data_bytes - bytes) {
        return aotx_gguf_read(file, offset, bytes, buffer); // refuses, with the message
    }
    unsigned char *out = static_cast<unsigned char *>(buffer);
    std::vector<int> codes((size_t)slices, 0);
    std::vector<std::thread> workers;
    const uint64_t each = (bytes / slices + 4095ull) & ~4095ull; // page-sized cuts
    auto part = [&](uint64_t index) {
        uint64_t begin = index * each;
        uint64_t end = index + 1 == slices ? bytes : (index + 1) * each;
        if (end > bytes) {
            end = bytes;
        }
        if (begin < end) {
            codes[(size_t)index] = aotx_gguf_read(file, offset + begin, end - begin, out + begin);
        }
    };
    uint64_t started = 1; // slice 0 runs on this thread
    try {
        workers.reserve((size_t)slices - 1);
        for (; started < slices; ++started) {
            workers.emplace_back(part, started);
        }
    } catch (...) {
        // no more threads to be had: the slices that did not start are read below
    }
    part(0);
    for (uint64_t i = started; i < slices; ++i) {
        part(i);
    }
    for (std::thread &worker : workers) {
        worker.join();
    }
    for (int code : codes) {
        if (code != 0) {
            return code;
        }
    }
    return AOTX_GGUF_OK;
}

extern "C" uint64_t aotx_gguf_row_bytes(uint32_t type, uint64_t row_weights)
{
    const BlockLayout *layout = layout_of(type);
    if (layout == nullptr || row_weights == 0 || (row_weights % layout->weights) != 0) {
        return 0;
    }
    if (row_weights / layout->weights > UINT64_MAX / layout->bytes) {
        return 0;
    }
    return row_weights / layout->weights * layout->bytes;
}

extern "C" int aotx_gguf_row_range(const aotx_gguf_tensor_info *info, uint64_t first_row, uint64_t rows,
                                   uint64_t *offset, uint64_t *bytes)
{
    if (info == nullptr || offset == nullptr || bytes == nullptr || info->dim_count == 0
        || info->dim_count > AOTX_GGUF_DIMS) {
        return 1;
    }
    const uint64_t row = aotx_gguf_row_bytes(info->type, info->dims[0]);
    if (row == 0 || info->bytes == 0 || (info->bytes % row) != 0) {
        return 1;
    }
    const uint64_t total = info->bytes / row;
    if (rows > total || first_row > total - rows) {
        return 1;
    }
    *offset = info->offset + first_row * row;
    *bytes = rows * row;
    return 0;
}
