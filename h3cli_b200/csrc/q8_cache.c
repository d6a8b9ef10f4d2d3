/* On-disk cache of packed q8 weights ("artifacts"), so that a checkpoint's bf16
 * matrices are quantised once and later loads are a single read into pinned memory.
 *
 * Behaviour follows h3cli's metadata-keyed quantisation cache
 * (src/weights/quant_cache.c:53-128): an artifact is identified by the canonical
 * path of the source file, its device/inode/size/mtime/ctime, the byte offset and
 * shape of the matrix, the scale group and the packing recipe -- never by hashing
 * weight bytes; a per-artifact lock file (flock) serialises writers; artifacts are
 * published with write-to-temporary + fsync + rename; an existing artifact whose
 * header or size does not match is an error, not a miss; the source is re-checked
 * before data is accepted or published.  The payload is the library's q8 blob:
 * int8 [rows, columns], zero padding to 16 bytes, fp32 scales, padded to 256. */
#define _GNU_SOURCE
#include "h3q8.h"
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/file.h>
#include <sys/stat.h>
#include <unistd.h>

#define CACHE_HEADER 128
#define CACHE_FORMAT 1u

struct h3q8_cache {
    char *source, *artifact;
    struct stat stamp;
    uint64_t offset, bytes, scale_offset;
    uint32_t rows, columns, group;
    unsigned char key[16];
    int lock;
};

static int refuse(char *error, size_t size, const char *what, const char *path) {
    if (error && size) snprintf(error, size, "%s: %s", what, path ? path : strerror(errno));
    return 0;
}
static void put_le(unsigned char *p, uint64_t v, unsigned bytes) {
    for (unsigned i = 0; i < bytes; i++) p[i] = (unsigned char)(v >> (8 * i));
}
static int same_file(const struct stat *a, const struct stat *b) {
    return S_ISREG(b->st_mode) && a->st_dev == b->st_dev && a->st_ino == b->st_ino && a->st_size == b->st_size &&
           a->st_mtim.tv_sec == b->st_mtim.tv_sec && a->st_mtim.tv_nsec == b->st_mtim.tv_nsec &&
           a->st_ctim.tv_sec == b->st_ctim.tv_sec && a->st_ctim.tv_nsec == b->st_ctim.tv_nsec;
}
static int transfer(int fd, void *data, size_t bytes, int writing) {
    unsigned char *p = data;
    while (bytes) {
        ssize_t n = writing ? write(fd, p, bytes) : read(fd, p, bytes);
        if (n < 0 && errno == EINTR) continue;
        if (n <= 0) return 0;
        p += (size_t)n;
        bytes -= (size_t)n;
    }
    return 1;
}
/* 128-bit FNV-1a style digest of the identity record: two 64-bit lanes with different offsets. */
static void digest(const unsigned char *data, size_t bytes, unsigned char out[16]) {
    uint64_t a = 0xcbf29ce484222325ull, b = 0x84222325cbf29ce4ull;
    for (size_t i = 0; i < bytes; i++) {
        a = (a ^ data[i]) * 0x100000001b3ull;
        b = (b ^ (data[i] + (unsigned char)(i * 31u))) * 0x100000001b3ull;
        b ^= a >> 29;
    }
    put_le(out, a, 8);
    put_le(out + 8, b, 8);
}
static void make_header(const h3q8_cache *c, unsigned char h[CACHE_HEADER]) {
    memset(h, 0, CACHE_HEADER);
    memcpy(h, "H3Q8ART1", 8);
    put_le(h + 8, CACHE_FORMAT, 4);
    put_le(h + 12, H3_Q8_VERSION, 4);
    put_le(h + 16, c->group, 4);
    put_le(h + 20, c->rows, 4);
    put_le(h + 24, c->columns, 4);
    put_le(h + 32, c->bytes, 8);
    put_le(h + 40, c->scale_offset, 8);
    put_le(h + 48, c->offset, 8);
    memcpy(h + 56, c->key, 16);
}

int h3q8_cache_unchanged(const h3q8_cache *c, char *error, size_t size) {
    struct stat now;
    if (!c || stat(c->source, &now) || !same_file(&c->stamp, &now))
        return refuse(error, size, "q8 source changed during loading/preparation; retry", c ? c->source : NULL);
    return 1;
}

void h3q8_cache_close(h3q8_cache *c) {
    if (!c) return;
    if (c->lock >= 0) { flock(c->lock, LOCK_UN); close(c->lock); }
    free(c->source);
    free(c->artifact);
    free(c);
}

h3q8_cache *h3q8_cache_open(const char *directory, const char *source, uint64_t offset, uint32_t rows, uint32_t columns,
                            uint32_t group, char *error, size_t size) {
    h3q8_cache *c = calloc(1, sizeof *c);
    if (!c) { refuse(error, size, "cannot allocate q8 cache entry", NULL); return NULL; }
    c->lock = -1;
    size_t scale_offset = 0, bytes = h3q8_q8_blob_bytes(rows, columns, group, &scale_offset);
    if (!directory || !*directory || !source || !bytes || (offset & 1)) {
        refuse(error, size, "invalid q8 cache arguments", source);
        goto failed;
    }
    c->source = realpath(source, NULL);
    if (!c->source || stat(c->source, &c->stamp) || !S_ISREG(c->stamp.st_mode) || offset > (uint64_t)c->stamp.st_size ||
        (uint64_t)rows * columns * 2 > (uint64_t)c->stamp.st_size - offset) {
        refuse(error, size, "invalid q8 source range", source);
        goto failed;
    }
    c->offset = offset; c->rows = rows; c->columns = columns; c->group = group;
    c->bytes = bytes; c->scale_offset = scale_offset;
    {
        /* identity: format, recipe, geometry, source file identity and times, then the canonical path */
        const uint64_t values[] = {CACHE_FORMAT, H3_Q8_VERSION, group, rows, columns, offset, (uint64_t)c->stamp.st_dev,
                                   (uint64_t)c->stamp.st_ino, (uint64_t)c->stamp.st_size, (uint64_t)c->stamp.st_mtim.tv_sec,
                                   (uint64_t)c->stamp.st_mtim.tv_nsec, (uint64_t)c->stamp.st_ctim.tv_sec,
                                   (uint64_t)c->stamp.st_ctim.tv_nsec, bytes};
        size_t path = strlen(c->source) + 1, total = sizeof values + path;
        unsigned char *identity = malloc(total);
        if (!identity) { refuse(error, size, "cannot allocate q8 cache identity", NULL); goto failed; }
        for (size_t i = 0; i < sizeof values / sizeof *values; i++) put_le(identity + 8 * i, values[i], 8);
        memcpy(identity + sizeof values, c->source, path);
        digest(identity, total, c->key);
        free(identity);
    }
    char hex[33];
    for (int i = 0; i < 16; i++) snprintf(hex + 2 * i, 3, "%02x", c->key[i]);
    char *lock = NULL;
    if (asprintf(&c->artifact, "%s/q8-v%u-g%u-%ux%u-%s.h3q8", directory, CACHE_FORMAT, group, rows, columns, hex) < 0) c->artifact = NULL;
    if (!c->artifact || asprintf(&lock, "%s.lock", c->artifact) < 0) {
        refuse(error, size, "cannot allocate q8 cache path", source);
        goto failed;
    }
    c->lock = open(lock, O_CREAT | O_RDWR, 0600);
    free(lock);
    if (c->lock < 0 || flock(c->lock, LOCK_EX)) { refuse(error, size, "cannot lock q8 artifact", c->artifact); goto failed; }
    if (!h3q8_cache_unchanged(c, error, size)) goto failed;
    return c;
failed:
    h3q8_cache_close(c);
    return NULL;
}

size_t h3q8_cache_payload_bytes(const h3q8_cache *c) { return c ? (size_t)c->bytes : 0; }
const char *h3q8_cache_artifact(const h3q8_cache *c) { return c ? c->artifact : NULL; }

/* 1 hit, 0 absent, -1 invalid: a malformed artifact never falls through to preparation. */
int h3q8_cache_read(h3q8_cache *c, void *payload, char *error, size_t size) {
    if (!c || !payload) return -1;
    int fd = open(c->artifact, O_RDONLY);
    if (fd < 0) {
        if (errno == ENOENT) return h3q8_cache_unchanged(c, error, size) ? 0 : -1;
        refuse(error, size, "cannot read q8 artifact", c->artifact);
        return -1;
    }
    struct stat before, after;
    unsigned char wanted[CACHE_HEADER], actual[CACHE_HEADER];
    make_header(c, wanted);
    int ok = !fstat(fd, &before) && S_ISREG(before.st_mode) && (uint64_t)before.st_size == CACHE_HEADER + c->bytes &&
             transfer(fd, actual, sizeof actual, 0) && !memcmp(actual, wanted, sizeof actual) &&
             transfer(fd, payload, (size_t)c->bytes, 0) && !fstat(fd, &after) && same_file(&before, &after);
    close(fd);
    if (!ok) {
        refuse(error, size, "corrupt or incompatible q8 artifact; remove it and prepare again", c->artifact);
        return -1;
    }
    return h3q8_cache_unchanged(c, error, size) ? 1 : -1;
}

int h3q8_cache_write(h3q8_cache *c, const void *payload, char *error, size_t size) {
    if (!c || !payload) return 0;
    if (!h3q8_cache_unchanged(c, error, size)) return 0;
    char *temporary = NULL;
    if (asprintf(&temporary, "%s.tmp.XXXXXX", c->artifact) < 0) return refuse(error, size, "cannot allocate q8 staging path", c->artifact);
    int fd = mkstemp(temporary);
    unsigned char h[CACHE_HEADER];
    make_header(c, h);
    int ok = fd >= 0;
    if (ok) {
        ok = transfer(fd, h, sizeof h, 1) && transfer(fd, (void *)payload, (size_t)c->bytes, 1) && !fsync(fd);
        if (close(fd)) ok = 0;
    }
    if (ok) ok = h3q8_cache_unchanged(c, error, size);
    if (ok) ok = !rename(temporary, c->artifact);
    if (!ok) {
        unlink(temporary);
        refuse(error, size, "cannot publish q8 artifact (source changed or I/O failure)", c->artifact);
    }
    free(temporary);
    return ok;
}
