// COLD persistence of the device pool: the reference's EventLog (scirust/src/eventlog.rs), an
// append-only file of evicted tiles -- 16-byte header (magic "SLLG", version 2, tile size 128,
// reserved 0) followed by 144-byte records (u64 seq, u32 slot, u32 FNV-1a checksum over seq, slot
// and tile, 128 tile bytes), little-endian, no timestamps: the same evictions give the same bytes.
// The pool lives in HBM, so an eviction first brings (seq, tile) of the slots that are about to go
// COLD to the host, appends their records in eviction order (ccos.rs:404-438), and only then flips
// the slots; with "require durable" a record that cannot be written (and fsync'ed) keeps its slot
// and all later ones live, as ElasticKvCache::evict does.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <memory>
#include <string>
#include <cstring>
#include <vector>

#include "pool.cuh"

namespace slha {

namespace {
constexpr uint32_t LOG_MAGIC = 0x534C4C47u;
constexpr size_t LOG_HEADER = 16, LOG_RECORD = 144;

void put32(unsigned char* p, uint32_t v) { for (int i = 0; i < 4; ++i) p[i] = (unsigned char)(v >> (8 * i)); }
void put64(unsigned char* p, uint64_t v) { for (int i = 0; i < 8; ++i) p[i] = (unsigned char)(v >> (8 * i)); }
uint32_t get32(const unsigned char* p) { return (uint32_t)p[0] | (uint32_t)p[1] << 8 | (uint32_t)p[2] << 16 | (uint32_t)p[3] << 24; }
uint64_t get64(const unsigned char* p) { return (uint64_t)get32(p) | (uint64_t)get32(p + 4) << 32; }

// record_checksum, eventlog.rs:146-169
uint32_t record_checksum(const unsigned char* seq_slot_12, const unsigned char* tile) {
    uint32_t h = 0x811C9DC5u;
    for (int i = 0; i < 12; ++i) h = (h ^ seq_slot_12[i]) * 0x01000193u;
    for (int i = 0; i < 128; ++i) h = (h ^ tile[i]) * 0x01000193u;
    return h;
}
Status io_error(const std::string& what) { return Status(SLHA_ERR_IO, "EventLog: " + what + ": " + std::strerror(errno)); }
}  // namespace

struct EventLog {
    int fd = -1;
    uint64_t records = 0;
    uint32_t version = 2;
    bool writable = true;
    ~EventLog() {
        if (fd >= 0) ::close(fd);
    }
};

void eventlog_close(EventLog* log) { delete log; }
uint64_t eventlog_records(const EventLog* log) { return log->records; }

// mode 0: create (truncate), 1: create only if absent, 2: open strictly, 3: open and drop one partial record at the tail,
// 4: open read-only  (EventLog::create / create_new / open / open_recover / open_read_only, eventlog.rs:186-300)
Status eventlog_open(const char* path, int mode, EventLog** out) {
    auto log = std::make_unique<EventLog>();
    if (mode == 0 || mode == 1) {
        log->fd = ::open(path, O_RDWR | O_CREAT | (mode == 1 ? O_EXCL : O_TRUNC), 0644);
        if (log->fd < 0) return io_error(std::string("cannot create ") + path);
        unsigned char h[LOG_HEADER] = {0};
        put32(h, LOG_MAGIC);
        put32(h + 4, 2);
        put32(h + 8, 128);
        if (::write(log->fd, h, LOG_HEADER) != (ssize_t)LOG_HEADER) return io_error("cannot write the header");
        *out = log.release();
        return Status();
    }
    if (mode < 2 || mode > 4) return Status(SLHA_ERR_DIMENSION, "EventLog: unknown open mode");
    log->writable = mode != 4;
    log->fd = ::open(path, log->writable ? O_RDWR : O_RDONLY);
    if (log->fd < 0) return io_error(std::string("cannot open ") + path);
    struct stat st;
    if (fstat(log->fd, &st) != 0) return io_error("fstat");
    uint64_t len = (uint64_t)st.st_size;
    if (len < LOG_HEADER) return Status(SLHA_ERR_IO, "EventLog: file shorter than header");
    unsigned char h[LOG_HEADER];
    if (::pread(log->fd, h, LOG_HEADER, 0) != (ssize_t)LOG_HEADER) return io_error("cannot read the header");
    if (get32(h) != LOG_MAGIC) return Status(SLHA_ERR_IO, "EventLog: bad magic");
    log->version = get32(h + 4);
    if (log->version != 1 && log->version != 2) return Status(SLHA_ERR_IO, "EventLog: unsupported version");
    if (get32(h + 8) != 128) return Status(SLHA_ERR_IO, "EventLog: tile-size mismatch");
    const uint64_t rem = (len - LOG_HEADER) % LOG_RECORD;
    if (rem) {
        if (mode != 3) return Status(SLHA_ERR_IO, "EventLog: truncated record");
        len -= rem;
        if (ftruncate(log->fd, (off_t)len) != 0 || fsync(log->fd) != 0) return io_error("cannot drop the partial record");
    }
    log->records = (len - LOG_HEADER) / LOG_RECORD;
    if (log->version == 2) {
        unsigned char r[LOG_RECORD];
        for (uint64_t i = 0; i < log->records; ++i) {
            if (::pread(log->fd, r, LOG_RECORD, (off_t)(LOG_HEADER + i * LOG_RECORD)) != (ssize_t)LOG_RECORD) return io_error("cannot read a record");
            if (get32(r + 12) != record_checksum(r, r + 16)) return Status(SLHA_ERR_IO, "EventLog: checksum mismatch in record " + std::to_string(i));
        }
    }
    *out = log.release();
    return Status();
}

// EventLog::append / append_durable (eventlog.rs:330-390): on failure the previous length is restored.
Status eventlog_append(EventLog* log, uint64_t seq, uint32_t slot, const unsigned char* tile, bool durable) {
    if (!log->writable) return Status(SLHA_ERR_IO, "EventLog: opened read-only");
    unsigned char r[LOG_RECORD];
    put64(r, seq);
    put32(r + 8, slot);
    std::memcpy(r + 16, tile, 128);
    put32(r + 12, log->version >= 2 ? record_checksum(r, r + 16) : 0u);
    const off_t at = (off_t)(LOG_HEADER + log->records * LOG_RECORD);
    const ssize_t w = ::pwrite(log->fd, r, LOG_RECORD, at);
    if (w != (ssize_t)LOG_RECORD || (durable && fsync(log->fd) != 0)) {
        const Status st = io_error("cannot append a record");
        if (ftruncate(log->fd, at) != 0) { /* nothing more can be done: the next open_recover drops the tail */ }
        return st;
    }
    ++log->records;
    return Status();
}

// The records of one eviction phase in one write (and, durable, one fsync): `*written` receives the number of leading
// records that are in the file afterwards -- all of them, or, when the write fell short or failed, the complete records
// that made it (the file is cut back to the last complete record; durable: to where it was, a batch is durable as a
// whole or not at all).  The records' order and bytes are those of n single appends.
Status eventlog_append_batch(EventLog* log, uint64_t n, const uint64_t* seq, const uint32_t* slot, const unsigned char* tiles,
                             bool durable, uint64_t* written) {
    *written = 0;
    if (n == 0) return Status();
    if (!log->writable) return Status(SLHA_ERR_IO, "EventLog: opened read-only");
    std::vector<unsigned char> buf((size_t)n * LOG_RECORD);
    for (uint64_t i = 0; i < n; ++i) {
        unsigned char* r = buf.data() + (size_t)i * LOG_RECORD;
        put64(r, seq[i]);
        put32(r + 8, slot[i]);
        std::memcpy(r + 16, tiles + (size_t)i * 128, 128);
        put32(r + 12, log->version >= 2 ? record_checksum(r, r + 16) : 0u);
    }
    const off_t at = (off_t)(LOG_HEADER + log->records * LOG_RECORD);
    size_t done = 0;
    bool failed = false;
    while (done < buf.size()) {
        const ssize_t w = ::pwrite(log->fd, buf.data() + done, buf.size() - done, at + (off_t)done);
        if (w <= 0) {
            failed = true;
            break;
        }
        done += (size_t)w;
    }
    if (!failed && durable && fsync(log->fd) != 0) {
        failed = true;
        done = 0;
    }
    if (failed) {
        const Status st = io_error("cannot append records");
        const uint64_t whole = done / LOG_RECORD;
        if (ftruncate(log->fd, at + (off_t)(whole * LOG_RECORD)) != 0) { /* the next open_recover drops the tail */ }
        log->records += whole;
        *written = whole;
        return st;
    }
    log->records += n;
    *written = n;
    return Status();
}

// EventLog::fetch_by_seq (eventlog.rs:475-477): the most recently appended record with that seq.
Status eventlog_fetch_by_seq(EventLog* log, uint64_t seq, bool* found, uint32_t* slot, unsigned char* tile) {
    *found = false;
    unsigned char r[LOG_RECORD];
    for (uint64_t i = log->records; i-- > 0;) {
        if (::pread(log->fd, r, LOG_RECORD, (off_t)(LOG_HEADER + i * LOG_RECORD)) != (ssize_t)LOG_RECORD) return io_error("cannot read a record");
        if (get64(r) != seq) continue;
        if (log->version >= 2 && get32(r + 12) != record_checksum(r, r + 16)) return Status(SLHA_ERR_IO, "EventLog: checksum mismatch");
        *found = true;
        *slot = get32(r + 8);
        std::memcpy(tile, r + 16, 128);
        return Status();
    }
    return Status();
}

}  // namespace slha
