// Training-state files for any architecture, readable by torch.load and by the reference host.
//
// The reference stores a checkpoint as an uncompressed PyTorch ZIP archive whose pickle names
// fifteen storages, and its reader (checkpoint.cpp:506-552) fetches them by record name:
// data/0 depth, data/1 context, data/2 weights, data/3 momentum, data/4 variance, data/5 step,
// data/6 total_steps, data/7-11 the OneCycle fractions, data/12 train_seconds, data/13
// final_loss_sums, data/14 final_loss_batches.  It knows only depth and context
// (checkpoint.cpp:164-166) and sizes everything from parameter_layout(depth), so a model of another
// width cannot be saved or loaded by it.  This writer keeps those fifteen records byte for byte
// where the reference expects them and adds data/15, "architecture": width, heads, hidden, norm,
// attention, mlp, tied, rope, hidden_optimizer.  A file of the reference architecture therefore
// still loads in the reference host; a file without data/15 (written by the reference host) loads
// here as the reference architecture.
#include "common.h"
#include <algorithm>
#include <climits>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>

namespace {
constexpr const char *SerializationId = "3407000000000000000000000000000000000000"; // what the reference reader requires
constexpr int ArchitectureFields = 9;

uint32_t crc32(const uint8_t *data, size_t size) {
    static uint32_t table[256];
    static bool ready = false;
    if (!ready) {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k)
                c = (c & 1) ? 0xedb88320u ^ (c >> 1) : c >> 1;
            table[i] = c;
        }
        ready = true;
    }
    uint32_t c = 0xffffffffu;
    for (size_t i = 0; i < size; ++i)
        c = table[(c ^ data[i]) & 0xff] ^ (c >> 8);
    return c ^ 0xffffffffu;
}

struct Bytes {
    std::vector<uint8_t> data;
    void u8(uint8_t v) { data.push_back(v); }
    void u16(uint16_t v) { u8(v & 0xff), u8(v >> 8); }
    void u32(uint32_t v) { u16(v & 0xffff), u16(v >> 16); }
    void raw(const void *p, size_t n) {
        const uint8_t *b = static_cast<const uint8_t *>(p);
        data.insert(data.end(), b, b + n);
    }
    void text(const std::string &s) { raw(s.data(), s.size()); }
};

// ---- pickle, protocol 2: only the opcodes a dict of tensors needs ----
struct Pickle : Bytes {
    void string(const std::string &s) { u8('X'), u32(uint32_t(s.size())), text(s); }      // BINUNICODE
    void global(const char *module, const char *name) { u8('c'), text(module), u8('\n'), text(name), u8('\n'); }
    void integer(uint32_t v) {                                                                // BININT1 / BININT
        if (v < 256)
            u8('K'), u8(uint8_t(v));
        else
            u8('J'), u32(v);
    }
    void open_dict() { u8('}'), u8('('); }        // EMPTY_DICT, MARK
    void close_dict() { u8('u'); }                // SETITEMS
    // key -> torch._utils._rebuild_tensor_v2(storage, 0, (count,), (1,), False, OrderedDict())
    void tensor(const std::string &key, const char *storage_type, int record, uint32_t count) {
        string(key);
        global("torch._utils", "_rebuild_tensor_v2");
        u8('(');                                  // arguments
        u8('(');                                  // persistent id: ('storage', type, key, location, count)
        string("storage");
        global("torch", storage_type);
        string(std::to_string(record));
        string("cpu");
        integer(count);
        u8('t'), u8('Q');                         // TUPLE, BINPERSID
        integer(0);                               // storage offset
        integer(count), u8(0x85);                 // size (count,)
        integer(1), u8(0x85);                     // stride (1,)
        u8(0x89);                                 // requires_grad False
        global("collections", "OrderedDict"), u8(')'), u8('R'); // backward hooks: OrderedDict()
        u8('t'), u8('R');                         // TUPLE, REDUCE
    }
};

// ---- ZIP, stored entries, payloads aligned to 64 bytes the way torch.save lays them out ----
struct Zip {
    Bytes out, directory;
    int entries = 0;
    void add(const std::string &name, const void *payload, size_t size) {
        if (size > 0xfffffff0ull || out.data.size() + size > 0xfffffff0ull)
            throw std::runtime_error("Checkpoint exceeds the 4 GB of a plain ZIP archive");
        const uint32_t crc = crc32(static_cast<const uint8_t *>(payload), size);
        const uint32_t local = uint32_t(out.data.size());
        size_t header = 30 + name.size() + 4; // with an empty extra field of 4 bytes
        const uint16_t pad = uint16_t((64 - (local + header) % 64) % 64);
        out.u32(0x04034b50), out.u16(0), out.u16(0), out.u16(0), out.u16(0), out.u16(0x21); // stored, 1980-01-01
        out.u32(crc), out.u32(uint32_t(size)), out.u32(uint32_t(size));
        out.u16(uint16_t(name.size())), out.u16(uint16_t(4 + pad));
        out.text(name);
        out.u16(0x4246), out.u16(pad); // extra field "FB" carrying the padding
        for (int i = 0; i < pad; ++i)
            out.u8('Z');
        out.raw(payload, size);
        directory.u32(0x02014b50), directory.u16(0), directory.u16(0), directory.u16(0), directory.u16(0);
        directory.u16(0), directory.u16(0x21);
        directory.u32(crc), directory.u32(uint32_t(size)), directory.u32(uint32_t(size));
        directory.u16(uint16_t(name.size())), directory.u16(0), directory.u16(0), directory.u16(0), directory.u16(0);
        directory.u32(0), directory.u32(local);
        directory.text(name);
        ++entries;
    }
    void add(const std::string &name, const std::string &textual) { add(name, textual.data(), textual.size()); }
    std::vector<uint8_t> finish() {
        const uint32_t start = uint32_t(out.data.size()), size = uint32_t(directory.data.size());
        out.raw(directory.data.data(), directory.data.size());
        out.u32(0x06054b50), out.u16(0), out.u16(0), out.u16(uint16_t(entries)), out.u16(uint16_t(entries));
        out.u32(size), out.u32(start), out.u16(0);
        return std::move(out.data);
    }
};

struct Record {
    size_t offset = 0, size = 0;
};
uint32_t get32(const std::vector<uint8_t> &a, size_t o) {
    if (o + 4 > a.size())
        throw std::runtime_error("Truncated checkpoint");
    return a[o] | a[o + 1] << 8 | a[o + 2] << 16 | uint32_t(a[o + 3]) << 24;
}
uint16_t get16(const std::vector<uint8_t> &a, size_t o) {
    if (o + 2 > a.size())
        throw std::runtime_error("Truncated checkpoint");
    return uint16_t(a[o] | a[o + 1] << 8);
}
std::map<std::string, Record> read_directory(const std::vector<uint8_t> &a) {
    if (a.size() < 22)
        throw std::runtime_error("Truncated checkpoint");
    size_t end = a.size() - 22;
    while (get32(a, end) != 0x06054b50) {
        if (end == 0)
            throw std::runtime_error("Checkpoint has no ZIP directory");
        --end;
    }
    const int entries = get16(a, end + 10);
    size_t at = get32(a, end + 16);
    std::map<std::string, Record> records;
    for (int i = 0; i < entries; ++i) {
        if (get32(a, at) != 0x02014b50)
            throw std::runtime_error("Invalid checkpoint directory entry");
        const uint16_t method = get16(a, at + 10);
        const uint32_t crc = get32(a, at + 16), packed = get32(a, at + 20), size = get32(a, at + 24);
        const uint16_t name_size = get16(a, at + 28), extra = get16(a, at + 30), comment = get16(a, at + 32);
        const size_t local = get32(a, at + 42);
        if (method != 0 || packed != size)
            throw std::runtime_error("Compressed checkpoint entries are not supported");
        if (at + 46 + name_size > a.size() || get32(a, local) != 0x04034b50)
            throw std::runtime_error("Invalid checkpoint entry");
        const std::string name(reinterpret_cast<const char *>(a.data() + at + 46), name_size);
        Record r;
        r.offset = local + 30 + get16(a, local + 26) + get16(a, local + 28);
        r.size = size;
        if (r.offset + r.size > a.size())
            throw std::runtime_error("Truncated checkpoint record " + name);
        if (crc32(a.data() + r.offset, r.size) != crc)
            throw std::runtime_error("Checkpoint record " + name + " fails its checksum");
        records[name] = r;
        at += 46 + size_t(name_size) + extra + comment;
    }
    return records;
}

// The host averages the loss over the last hundredth of the schedule (at least one step); a state can
// hold at most as many summed batches as steps of that window are done (checkpoint.cpp:450-454).
uint64_t loss_window_batches_done(uint64_t step, int64_t total_steps) {
    const int64_t window = std::max<int64_t>(1, (total_steps + 99) / 100);
    const int64_t first = std::max<int64_t>(0, total_steps - window);
    return uint64_t(std::max<int64_t>(0, int64_t(step) - first));
}

void architecture_of(const TgConfigEx &c, int64_t (&fields)[ArchitectureFields]) {
    const int64_t values[ArchitectureFields] = {c.width, c.heads, c.hidden, c.norm, c.attention,
                                                c.mlp,   c.tied,  c.rope,   c.hidden_optimizer};
    memcpy(fields, values, sizeof(values));
}
} // namespace

void save_checkpoint(const std::string &path, const TgConfigEx &c, const TgCheckpoint &s) {
    validate_config(c);
    const int64_t count = make_layout(c).count;
    const int context = c.base.context;
    if (!s.weights || !s.momentum || !s.variance || !s.final_loss_sums)
        throw std::runtime_error("Checkpoint state is incomplete");
    if (s.scheduler.total_steps < 1 || s.step > uint64_t(s.scheduler.total_steps))
        throw std::runtime_error("Invalid checkpoint scheduler state");
    if (s.final_loss_batches > loss_window_batches_done(s.step, s.scheduler.total_steps))
        throw std::runtime_error("Invalid checkpoint final loss state");
    onecycle_point(s.scheduler, 0);

    Pickle p;
    p.u8(0x80), p.u8(2);
    p.open_dict();
    p.string("model"), p.open_dict();
    p.tensor("depth", "LongStorage", 0, 1);
    p.tensor("context", "LongStorage", 1, 1);
    p.tensor("weights", "FloatStorage", 2, uint32_t(count));
    p.tensor("architecture", "LongStorage", 15, ArchitectureFields);
    p.close_dict();
    p.string("opt"), p.open_dict();
    p.tensor("momentum", "FloatStorage", 3, uint32_t(count));
    p.tensor("variance", "FloatStorage", 4, uint32_t(count));
    p.tensor("step", "LongStorage", 5, 1);
    p.close_dict();
    p.string("lr_scheduler"), p.open_dict();
    p.tensor("total_steps", "LongStorage", 6, 1);
    p.tensor("step", "LongStorage", 5, 1);
    p.tensor("warmup_fraction", "DoubleStorage", 7, 1);
    p.tensor("initial_lr_fraction", "DoubleStorage", 8, 1);
    p.tensor("final_lr_fraction", "DoubleStorage", 9, 1);
    p.tensor("low_momentum", "DoubleStorage", 10, 1);
    p.tensor("high_momentum", "DoubleStorage", 11, 1);
    p.close_dict();
    p.string("trainer"), p.open_dict();
    p.tensor("train_seconds", "DoubleStorage", 12, 1);
    p.tensor("final_loss_sums", "DoubleStorage", 13, uint32_t(context));
    p.tensor("final_loss_batches", "LongStorage", 14, 1);
    p.close_dict();
    p.close_dict();
    p.u8('.');

    Zip zip;
    const std::string prefix = "archive/";
    zip.add(prefix + "data.pkl", p.data.data(), p.data.size());
    zip.add(prefix + ".format_version", std::string("2"));
    zip.add(prefix + ".storage_alignment", std::string("64"));
    zip.add(prefix + "byteorder", std::string("little"));
    auto scalar = [&](int record, int64_t v) { zip.add(prefix + "data/" + std::to_string(record), &v, 8); };
    auto real = [&](int record, double v) { zip.add(prefix + "data/" + std::to_string(record), &v, 8); };
    scalar(0, c.base.depth);
    scalar(1, context);
    zip.add(prefix + "data/2", s.weights, size_t(count) * 4);
    zip.add(prefix + "data/3", s.momentum, size_t(count) * 4);
    zip.add(prefix + "data/4", s.variance, size_t(count) * 4);
    scalar(5, int64_t(s.step));
    scalar(6, s.scheduler.total_steps);
    real(7, s.scheduler.warmup_fraction);
    real(8, s.scheduler.initial_lr_fraction);
    real(9, s.scheduler.final_lr_fraction);
    real(10, s.scheduler.low_momentum);
    real(11, s.scheduler.high_momentum);
    real(12, s.train_seconds);
    zip.add(prefix + "data/13", s.final_loss_sums, size_t(context) * 8);
    scalar(14, int64_t(s.final_loss_batches));
    int64_t fields[ArchitectureFields];
    architecture_of(c, fields);
    zip.add(prefix + "data/15", fields, sizeof(fields));
    zip.add(prefix + "version", std::string("3\n"));
    zip.add(prefix + ".data/serialization_id", std::string(SerializationId));
    const std::vector<uint8_t> archive = zip.finish();

    // Written beside the target and moved into place, so a crash never leaves half a checkpoint.
    const std::string staged = path + ".tmp";
    {
        std::ofstream file(staged, std::ios::binary | std::ios::trunc);
        file.write(reinterpret_cast<const char *>(archive.data()), std::streamsize(archive.size()));
        file.close();
        if (!file)
            throw std::runtime_error("Cannot write checkpoint " + staged);
    }
    if (std::rename(staged.c_str(), path.c_str()) != 0)
        throw std::runtime_error("Cannot move checkpoint into place at " + path);
}

void load_checkpoint(const std::string &path, const TgConfigEx &c, TgCheckpoint &s) {
    validate_config(c);
    const int64_t count = make_layout(c).count;
    const int context = c.base.context;
    if (!s.weights || !s.momentum || !s.variance || !s.final_loss_sums)
        throw std::runtime_error("Checkpoint destination is incomplete");
    std::ifstream file(path, std::ios::binary);
    if (!file)
        throw std::runtime_error("Cannot open checkpoint " + path);
    const std::vector<uint8_t> a((std::istreambuf_iterator<char>(file)), std::istreambuf_iterator<char>());
    const auto records = read_directory(a);
    std::string prefix;
    for (const auto &entry : records) {
        const std::string suffix = "/data.pkl";
        if (entry.first.size() > suffix.size() &&
            entry.first.compare(entry.first.size() - suffix.size(), suffix.size(), suffix) == 0)
            prefix = entry.first.substr(0, entry.first.size() - suffix.size() + 1);
    }
    if (prefix.empty())
        throw std::runtime_error("Checkpoint has no data.pkl");
    auto find = [&](const std::string &name, size_t bytes) {
        auto found = records.find(prefix + name);
        if (found == records.end())
            throw std::runtime_error("Checkpoint lacks record " + name);
        if (found->second.size != bytes)
            throw std::runtime_error("Checkpoint record " + name + " has " + std::to_string(found->second.size) +
                                     " bytes, this model needs " + std::to_string(bytes));
        return a.data() + found->second.offset;
    };
    auto scalar = [&](int record) {
        int64_t v;
        memcpy(&v, find("data/" + std::to_string(record), 8), 8);
        return v;
    };
    auto real = [&](int record) {
        double v;
        memcpy(&v, find("data/" + std::to_string(record), 8), 8);
        return v;
    };
    if (scalar(0) != c.base.depth || scalar(1) != context)
        throw std::runtime_error("Checkpoint architecture mismatch");
    int64_t expected[ArchitectureFields];
    architecture_of(c, expected);
    if (records.count(prefix + "data/15")) {
        int64_t stored[ArchitectureFields];
        memcpy(stored, find("data/15", sizeof(stored)), sizeof(stored));
        if (memcmp(stored, expected, sizeof(stored)) != 0)
            throw std::runtime_error("Checkpoint architecture mismatch");
    } else { // a file of the reference host: the reference architecture and nothing else
        const int64_t reference[ArchitectureFields] = {16, 4, 48, TG_NORM_RMS, TG_ATTENTION_ARGMAX, TG_MLP_SWIGLU,
                                                       0,  TG_ROPE_PARTIAL, TG_HIDDEN_MUON};
        if (memcmp(reference, expected, sizeof(reference)) != 0)
            throw std::runtime_error("Checkpoint architecture mismatch");
    }
    memcpy(s.weights, find("data/2", size_t(count) * 4), size_t(count) * 4);
    memcpy(s.momentum, find("data/3", size_t(count) * 4), size_t(count) * 4);
    memcpy(s.variance, find("data/4", size_t(count) * 4), size_t(count) * 4);
    s.step = uint64_t(scalar(5));
    const int64_t total = scalar(6);
    if (total < 1 || total > INT_MAX || s.step > uint64_t(total))
        throw std::runtime_error("Invalid checkpoint scheduler state");
    s.scheduler = TgOneCycle{};
    s.scheduler.total_steps = int(total);
    s.scheduler.warmup_fraction = real(7);
    s.scheduler.initial_lr_fraction = real(8);
    s.scheduler.final_lr_fraction = real(9);
    s.scheduler.low_momentum = real(10);
    s.scheduler.high_momentum = real(11);
    s.train_seconds = real(12);
    memcpy(s.final_loss_sums, find("data/13", size_t(context) * 8), size_t(context) * 8);
    s.final_loss_batches = uint64_t(scalar(14));
    if (s.final_loss_batches > loss_window_batches_done(s.step, s.scheduler.total_steps))
        throw std::runtime_error("Invalid checkpoint final loss state");
    onecycle_point(s.scheduler, 0);
}
