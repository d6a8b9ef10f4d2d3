/* On-disk artifacts of packed q8 weights: a checkpoint's bf16 matrices are quantised once, and
 * every later load is one positional read into pinned memory.
 *
 * What the protocol has in common with h3cli's quantisation cache (src/weights/quant_cache.h:14-41,
 * strict mode src/cuda/cuda_quant.cuh:186-256) are its guarantees, because callers rely on them:
 *   - an artifact is found by a key, never by trusting a file name a user could have copied:
 *       metadata kind  SHA-256 over (format, recipe, geometry, offset, the source file's identity and
 *                      timestamps, its canonical path) -- no weight byte is read to open a hit;
 *       content kind   SHA-256 over the geometry and the source matrix bytes themselves, and the
 *                      artifact carries a SHA-256 of its payload that every read verifies;
 *   - one preparer at a time: an exclusive flock on "<artifact>.lock" from open to close;
 *   - publication is all or nothing: temporary file, fsync, rename, fsync of the directory;
 *   - a file that exists but does not match is an ERROR ("remove it and prepare again"), never a miss
 *     that would be silently re-prepared over;
 *   - the source is re-examined before a hit is accepted and before an artifact is published.
 *
 * Layout: a 128-byte header written and compared as one struct, then the library's q8 blob
 * (int8 [rows, columns], zero padding to 16 bytes, fp32 scales, padded to 256 bytes).
 */
#define _GNU_SOURCE
#include "h3q8.h"
#include <errno.h>
#include <fcntl.h>
#include <libgen.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/file.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

/* ------------------------------------------------------------------ SHA-256 (FIPS 180-4) */
typedef struct { uint32_t state[8]; uint64_t length; unsigned char block[64]; size_t filled; } sha256;

static const uint32_t SHA_K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be,
    0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa,
    0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85,
    0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3,
    0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f,
    0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

static uint32_t rotr(uint32_t v, unsigned n) { return (v >> n) | (v << (32 - n)); }

static void sha256_block(sha256 *s, const unsigned char *p) {
    uint32_t w[64], v[8];
    for (int i = 0; i < 16; i++) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; i++)
        w[i] = w[i - 16] + (rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3)) + w[i - 7] +
               (rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10));
    memcpy(v, s->state, sizeof v);
    for (int i = 0; i < 64; i++) {
        const uint32_t t1 = v[7] + (rotr(v[4], 6) ^ rotr(v[4], 11) ^ rotr(v[4], 25)) + ((v[4] & v[5]) ^ (~v[4] & v[6])) + SHA_K[i] + w[i];
        const uint32_t t2 = (rotr(v[0], 2) ^ rotr(v[0], 13) ^ rotr(v[0], 22)) + ((v[0] & v[1]) ^ (v[0] & v[2]) ^ (v[1] & v[2]));
        memmove(v + 1, v, 7 * sizeof v[0]);
        v[4] += t1;
        v[0] = t1 + t2;
    }
    for (int i = 0; i < 8; i++) s->state[i] += v[i];
}
static void sha256_begin(sha256 *s) {
    static const uint32_t initial[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(s->state, initial, sizeof initial);
    s->length = 0;
    s->filled = 0;
}
static void sha256_add(sha256 *s, const void *data, size_t bytes) {
    const unsigned char *p = data;
    s->length += bytes;
    while (bytes) {
        if (!s->filled && bytes >= 64) { sha256_block(s, p); p += 64; bytes -= 64; continue; }
        size_t take = 64 - s->filled < bytes ? 64 - s->filled : bytes;
        memcpy(s->block + s->filled, p, take);
        s->filled += take; p += take; bytes -= take;
        if (s->filled == 64) { sha256_block(s, s->block); s->filled = 0; }
    }
}
static void sha256_end(sha256 *s, unsigned char out[32]) {
    const uint64_t bits = s->length * 8;
    unsigned char pad[72] = {0x80};
    size_t padding = (s->filled < 56 ? 56 : 120) - s->filled;
    for (int i = 0; i < 8; i++) pad[padding + i] = (unsigned char)(bits >> (56 - 8 * i));
    sha256_add(s, pad, padding + 8);
    for (int i = 0; i < 8; i++)
        for (int b = 0; b < 4; b++) out[4 * i + b] = (unsigned char)(s->state[i] >> (24 - 8 * b));
}
void h3q8_sha256(const void *data, size_t bytes, unsigned char out[32]) {
    sha256 s;
    sha256_begin(&s);
    sha256_add(&s, data, bytes);
    sha256_end(&s, out);
}

/* ------------------------------------------------------------------ the artifact */
enum { KIND_METADATA = 0, KIND_CONTENT = 1 };
#define ARTIFACT_FORMAT 2u

typedef struct {            /* exactly what is on disk in front of the payload; little-endian hosts */
    char magic[8];
    uint32_t format, recipe, kind, group, rows, columns;
    uint64_t payload_bytes, scale_offset, source_offset;
    unsigned char key[32];
    unsigned char payload_digest[32];   /* content kind; zero otherwise */
    unsigned char reserved[8];
} artifact_header;
_Static_assert(sizeof(artifact_header) == 128, "artifact header is 128 bytes");

typedef struct {            /* what identifies a source file without reading it */
    uint64_t device, inode, size, modified_s, modified_ns, changed_s, changed_ns;
} file_identity;

struct h3q8_cache {
    artifact_header expect;
    file_identity source_identity;
    uint64_t where;             /* byte offset of the matrix in the source file */
    char *source, *artifact;
    int lock;
};

static int say(char *error, size_t size, const char *what, const char *subject) {
    if (error && size) snprintf(error, size, "%s: %s", what, subject ? subject : strerror(errno));
    return 0;
}
static int identify(const char *path, file_identity *id) {
    struct stat st;
    if (stat(path, &st) || !S_ISREG(st.st_mode)) return 0;
    *id = (file_identity){(uint64_t)st.st_dev, (uint64_t)st.st_ino, (uint64_t)st.st_size, (uint64_t)st.st_mtim.tv_sec,
                          (uint64_t)st.st_mtim.tv_nsec, (uint64_t)st.st_ctim.tv_sec, (uint64_t)st.st_ctim.tv_nsec};
    return 1;
}
/* whole-range positional I/O: no file position is shared with anybody */
static int at(int fd, void *data, size_t bytes, off_t offset, int writing) {
    unsigned char *p = data;
    while (bytes) {
        ssize_t n = writing ? pwrite(fd, p, bytes, offset) : pread(fd, p, bytes, offset);
        if (n < 0 && errno == EINTR) continue;
        if (n <= 0) return 0;
        p += n; offset += n; bytes -= (size_t)n;
    }
    return 1;
}

int h3q8_cache_unchanged(const h3q8_cache *c, char *error, size_t size) {
    file_identity now;
    if (!c || !identify(c->source, &now) || memcmp(&now, &c->source_identity, sizeof now))
        return say(error, size, "q8 source changed during loading/preparation; retry", c ? c->source : NULL);
    return 1;
}

void h3q8_cache_close(h3q8_cache *c) {
    if (!c) return;
    if (c->lock >= 0) { flock(c->lock, LOCK_UN); close(c->lock); }
    free(c->source);
    free(c->artifact);
    free(c);
}

/* key of the content kind: geometry, then the matrix bytes as they lie in the file */
static int content_key(h3q8_cache *c, unsigned char key[32]) {
    const size_t bytes = (size_t)c->expect.rows * c->expect.columns * 2, page = (size_t)sysconf(_SC_PAGESIZE);
    const size_t lead = (size_t)(c->where % page);
    int fd = open(c->source, O_RDONLY);
    if (fd < 0) return 0;
    void *mapping = mmap(NULL, bytes + lead, PROT_READ, MAP_PRIVATE, fd, (off_t)(c->where - lead));
    close(fd);
    if (mapping == MAP_FAILED) return 0;
    sha256 s;
    sha256_begin(&s);
    const uint32_t geometry[5] = {ARTIFACT_FORMAT, H3_Q8_VERSION, c->expect.group, c->expect.rows, c->expect.columns};
    sha256_add(&s, geometry, sizeof geometry);
    sha256_add(&s, (const unsigned char *)mapping + lead, bytes);
    sha256_end(&s, key);
    munmap(mapping, bytes + lead);
    return 1;
}

static h3q8_cache *open_kind(int kind, const char *directory, const char *source, uint64_t offset, uint32_t rows, uint32_t columns,
                             uint32_t group, char *error, size_t size) {
    h3q8_cache *c = calloc(1, sizeof *c);
    if (!c) { say(error, size, "cannot allocate q8 cache entry", NULL); return NULL; }
    c->lock = -1;
    size_t scale_offset = 0;
    const size_t payload = h3q8_q8_blob_bytes(rows, columns, group, &scale_offset);
    char *lock_path = NULL;
    if (!directory || !*directory || !source || !payload || (offset & 1)) { say(error, size, "invalid q8 cache arguments", source); goto fail; }
    c->source = realpath(source, NULL);
    if (!c->source || !identify(c->source, &c->source_identity) || offset > c->source_identity.size ||
        (uint64_t)rows * columns * 2 > c->source_identity.size - offset) {
        say(error, size, "invalid q8 source range", source);
        goto fail;
    }
    memcpy(c->expect.magic, "H3Q8ART2", 8);
    c->expect.format = ARTIFACT_FORMAT; c->expect.recipe = H3_Q8_VERSION; c->expect.kind = (uint32_t)kind;
    c->expect.group = group; c->expect.rows = rows; c->expect.columns = columns;
    c->expect.payload_bytes = payload; c->expect.scale_offset = scale_offset;
    c->where = offset;
    c->expect.source_offset = kind == KIND_CONTENT ? 0 : offset;   /* where the bytes lay is no part of a content key */
    if (kind == KIND_CONTENT) {
        if (!content_key(c, c->expect.key)) { say(error, size, "cannot read q8 source for its content key", c->source); goto fail; }
    } else {
        sha256 s;
        sha256_begin(&s);
        sha256_add(&s, &c->expect, offsetof(artifact_header, key));          /* format, recipe, geometry, offset */
        sha256_add(&s, &c->source_identity, sizeof c->source_identity);      /* which file, and as of when        */
        sha256_add(&s, c->source, strlen(c->source) + 1);                    /* under which canonical name        */
        sha256_end(&s, c->expect.key);
    }
    char hex[65];
    for (int i = 0; i < 32; i++) snprintf(hex + 2 * i, 3, "%02x", c->expect.key[i]);
    if (asprintf(&c->artifact, "%s/q8-%s-g%u-%ux%u-%s.h3q8", directory, kind == KIND_CONTENT ? "content" : "meta", group, rows, columns, hex) < 0)
        c->artifact = NULL;
    if (!c->artifact || asprintf(&lock_path, "%s.lock", c->artifact) < 0) { lock_path = NULL; say(error, size, "cannot allocate q8 cache path", source); goto fail; }
    c->lock = open(lock_path, O_CREAT | O_RDWR | O_CLOEXEC, 0600);
    if (c->lock < 0 || flock(c->lock, LOCK_EX)) { say(error, size, "cannot lock q8 artifact", c->artifact); goto fail; }
    free(lock_path);
    if (!h3q8_cache_unchanged(c, error, size)) { h3q8_cache_close(c); return NULL; }
    return c;
fail:
    free(lock_path);
    h3q8_cache_close(c);
    return NULL;
}

h3q8_cache *h3q8_cache_open(const char *directory, const char *source, uint64_t offset, uint32_t rows, uint32_t columns,
                            uint32_t group, char *error, size_t size) {
    return open_kind(KIND_METADATA, directory, source, offset, rows, columns, group, error, size);
}
h3q8_cache *h3q8_cache_open_content(const char *directory, const char *source, uint64_t offset, uint32_t rows, uint32_t columns,
                                    uint32_t group, char *error, size_t size) {
    return open_kind(KIND_CONTENT, directory, source, offset, rows, columns, group, error, size);
}

size_t h3q8_cache_payload_bytes(const h3q8_cache *c) { return c ? (size_t)c->expect.payload_bytes : 0; }
const char *h3q8_cache_artifact(const h3q8_cache *c) { return c ? c->artifact : NULL; }

/* 1 hit, 0 absent, -1 invalid: a malformed artifact never falls through to preparation. */
int h3q8_cache_read(h3q8_cache *c, void *payload, char *error, size_t size) {
    if (!c || !payload) return -1;
    int fd = open(c->artifact, O_RDONLY | O_CLOEXEC);
    if (fd < 0) {
        if (errno == ENOENT) return h3q8_cache_unchanged(c, error, size) ? 0 : -1;
        say(error, size, "cannot read q8 artifact", c->artifact);
        return -1;
    }
    artifact_header found, wanted = c->expect;
    struct stat st;
    const size_t bytes = (size_t)c->expect.payload_bytes;
    int good = !fstat(fd, &st) && S_ISREG(st.st_mode) && (uint64_t)st.st_size == sizeof found + bytes && at(fd, &found, sizeof found, 0, 0);
    if (good && c->expect.kind == KIND_CONTENT) memcpy(wanted.payload_digest, found.payload_digest, sizeof wanted.payload_digest);
    good = good && !memcmp(&found, &wanted, sizeof found) && at(fd, payload, bytes, sizeof found, 0);
    if (good && c->expect.kind == KIND_CONTENT) {
        unsigned char digest[32];
        h3q8_sha256(payload, bytes, digest);
        good = !memcmp(digest, found.payload_digest, sizeof digest);
    }
    struct stat again;
    good = good && !fstat(fd, &again) && again.st_size == st.st_size && again.st_mtim.tv_sec == st.st_mtim.tv_sec &&
           again.st_mtim.tv_nsec == st.st_mtim.tv_nsec;
    close(fd);
    if (!good) {
        say(error, size, "corrupt or incompatible q8 artifact; remove it and prepare again", c->artifact);
        return -1;
    }
    return h3q8_cache_unchanged(c, error, size) ? 1 : -1;
}

int h3q8_cache_write(h3q8_cache *c, const void *payload, char *error, size_t size) {
    if (!c || !payload || !h3q8_cache_unchanged(c, error, size)) return 0;
    artifact_header header = c->expect;
    const size_t bytes = (size_t)c->expect.payload_bytes;
    if (c->expect.kind == KIND_CONTENT) h3q8_sha256(payload, bytes, header.payload_digest);
    char *staging = NULL;
    if (asprintf(&staging, "%s.tmp.XXXXXX", c->artifact) < 0) return say(error, size, "cannot allocate q8 staging path", c->artifact);
    int fd = mkostemp(staging, O_CLOEXEC);
    int good = fd >= 0 && at(fd, &header, sizeof header, 0, 1) && at(fd, (void *)payload, bytes, sizeof header, 1) && !fsync(fd);
    if (fd >= 0 && close(fd)) good = 0;
    good = good && h3q8_cache_unchanged(c, error, size) && !rename(staging, c->artifact);
    if (good) {   /* the rename itself must survive a crash too */
        char *copy = strdup(c->artifact);
        int dir = copy ? open(dirname(copy), O_RDONLY | O_DIRECTORY | O_CLOEXEC) : -1;
        if (dir >= 0) { fsync(dir); close(dir); }
        free(copy);
    } else {
        if (fd >= 0) unlink(staging);
        say(error, size, "cannot publish q8 artifact (source changed or I/O failure)", c->artifact);
    }
    free(staging);
    return good;
}
