/* h3q8_prepare: build the packed-weight artifacts of a transformer directory ahead of time,
 * with no encoder, denoising or VAE work -- the job of h3cli's src/weights/quant_prepare.c.
 *
 *   h3q8_prepare w8a16|w8a8 TRANSFORMER_DIRECTORY CACHE_DIRECTORY [SCALE_GROUP]
 *   h3q8_prepare list TRANSFORMER_DIRECTORY      (no GPU: prints name, rows, columns, byte offset)
 *
 * Every *.safetensors file of the directory is scanned; each 2-D BF16 tensor named
 * blocks.<n>.{attn.qkv_proj,attn.out_proj,mlp.fc1,mlp.fc2}.weight is passed to
 * h3_gpu_quant_load, which packs it on the GPU and publishes the artifact (or finds it
 * already there).  Shapes come from the file, not from a table, so any DiT width works;
 * rows and columns must be multiples of 128 as the loader requires.
 *
 * safetensors layout: u64 little-endian header length, a JSON object
 * {"name": {"dtype": "BF16", "shape": [rows, columns], "data_offsets": [begin, end]}, ...},
 * then the payload; offsets are relative to the end of the header. */
#define _GNU_SOURCE
#include "h3q8.h"
#include <dirent.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { const char *p, *end; int failed; } scan;

static void blanks(scan *s) { while (s->p < s->end && (*s->p == ' ' || *s->p == '\n' || *s->p == '\t' || *s->p == '\r')) s->p++; }
static int take(scan *s, char c) {
    blanks(s);
    if (s->p < s->end && *s->p == c) { s->p++; return 1; }
    return 0;
}
/* Copies a JSON string (escapes kept verbatim apart from \" and \\) into out. */
static int string(scan *s, char *out, size_t size) {
    size_t n = 0;
    if (!take(s, '"')) return s->failed = 1, 0;
    while (s->p < s->end && *s->p != '"') {
        char c = *s->p++;
        if (c == '\\' && s->p < s->end) c = *s->p++;
        if (out && n + 1 < size) out[n++] = c;
    }
    if (out && size) out[n] = 0;
    if (s->p >= s->end) return s->failed = 1, 0;
    s->p++;
    return 1;
}
static int number(scan *s, uint64_t *value) {
    blanks(s);
    const char *begin = s->p;
    uint64_t v = 0;
    while (s->p < s->end && *s->p >= '0' && *s->p <= '9') v = v * 10 + (uint64_t)(*s->p++ - '0');
    if (s->p == begin) return s->failed = 1, 0;
    *value = v;
    return 1;
}
static void skip_value(scan *s) {
    blanks(s);
    if (s->p >= s->end) { s->failed = 1; return; }
    if (*s->p == '"') { string(s, NULL, 0); return; }
    if (*s->p == '{' || *s->p == '[') {
        const char close = *s->p == '{' ? '}' : ']';
        const int object = *s->p == '{';
        s->p++;
        if (take(s, close)) return;
        do {
            if (object) { string(s, NULL, 0); if (!take(s, ':')) s->failed = 1; }
            skip_value(s);
        } while (!s->failed && take(s, ','));
        if (!take(s, close)) s->failed = 1;
        return;
    }
    while (s->p < s->end && *s->p != ',' && *s->p != '}' && *s->p != ']') s->p++; /* number, true, false, null */
}
static unsigned array(scan *s, uint64_t *values, unsigned capacity) {
    unsigned n = 0;
    if (!take(s, '[')) return s->failed = 1, 0;
    if (take(s, ']')) return 0;
    do {
        uint64_t v;
        if (!number(s, &v)) return 0;
        if (n < capacity) values[n] = v;
        n++;
    } while (take(s, ','));
    if (!take(s, ']')) s->failed = 1;
    return n;
}

typedef struct { char dtype[16]; uint64_t shape[4], offsets[2]; unsigned dims, bounds; } entry;

static void tensor_entry(scan *s, entry *e) {
    memset(e, 0, sizeof *e);
    if (!take(s, '{')) { s->failed = 1; return; }
    if (take(s, '}')) return;
    do {
        char key[32];
        if (!string(s, key, sizeof key) || !take(s, ':')) { s->failed = 1; return; }
        if (!strcmp(key, "dtype")) string(s, e->dtype, sizeof e->dtype);
        else if (!strcmp(key, "shape")) e->dims = array(s, e->shape, 4);
        else if (!strcmp(key, "data_offsets")) e->bounds = array(s, e->offsets, 2);
        else skip_value(s);
    } while (!s->failed && take(s, ','));
    if (!take(s, '}')) s->failed = 1;
}

/* blocks.<digits>.<one of the four projection names> */
static int wanted(const char *name) {
    static const char *const projections[] = {"attn.qkv_proj.weight", "attn.out_proj.weight", "mlp.fc1.weight", "mlp.fc2.weight"};
    if (strncmp(name, "blocks.", 7)) return 0;
    const char *p = name + 7;
    if (*p < '0' || *p > '9') return 0;
    while (*p >= '0' && *p <= '9') p++;
    if (*p++ != '.') return 0;
    for (unsigned i = 0; i < 4; i++) if (!strcmp(p, projections[i])) return 1;
    return 0;
}

static int prepare_file(h3_gpu *gpu, const char *path, unsigned *done, char *error, size_t size) {
    FILE *f = fopen(path, "rb");
    unsigned char prefix[8];
    if (!f || fread(prefix, 1, 8, f) != 8) {
        if (f) fclose(f);
        snprintf(error, size, "cannot read %s", path);
        return 0;
    }
    uint64_t length = 0;
    for (int i = 7; i >= 0; i--) length = (length << 8) | prefix[i];
    char *header = length && length < (UINT64_C(1) << 30) ? malloc((size_t)length) : NULL;
    if (!header || fread(header, 1, (size_t)length, f) != length) {
        fclose(f);
        free(header);
        snprintf(error, size, "invalid safetensors header in %s", path);
        return 0;
    }
    fclose(f);
    scan s = {header, header + length, 0};
    int ok = take(&s, '{');
    if (ok && !take(&s, '}')) do {
        char name[256];
        entry e;
        if (!string(&s, name, sizeof name) || !take(&s, ':')) { s.failed = 1; break; }
        if (!wanted(name)) { skip_value(&s); continue; }
        tensor_entry(&s, &e);
        if (s.failed) break;
        if (strcmp(e.dtype, "BF16") || e.dims != 2 || e.bounds != 2 || e.shape[0] > UINT32_MAX || e.shape[1] > UINT32_MAX ||
            e.offsets[1] < e.offsets[0] || e.offsets[1] - e.offsets[0] != e.shape[0] * e.shape[1] * 2) {
            snprintf(error, size, "missing/invalid %s in %s", name, path);
            ok = 0;
            break;
        }
        if (!gpu) {
            printf("%s %llu %llu %llu\n", name, (unsigned long long)e.shape[0], (unsigned long long)e.shape[1],
                   (unsigned long long)(8 + length + e.offsets[0]));
            ++*done;
            continue;
        }
        h3_gpu_tensor *weight = h3_gpu_quant_load(gpu, path, 8 + length + e.offsets[0], (uint32_t)e.shape[0], (uint32_t)e.shape[1]);
        if (!weight) {
            snprintf(error, size, "%s: %s", name, h3_gpu_error(gpu));
            ok = 0;
            break;
        }
        h3_gpu_tensor_free(weight);
        fprintf(stderr, "quantized weights %u: %s %llux%llu\n", ++*done, name, (unsigned long long)e.shape[0], (unsigned long long)e.shape[1]);
    } while (take(&s, ','));
    if (ok && s.failed) {
        snprintf(error, size, "malformed safetensors header in %s", path);
        ok = 0;
    }
    free(header);
    return ok;
}

static int by_name(const struct dirent **a, const struct dirent **b) { return strcmp((*a)->d_name, (*b)->d_name); }
static int is_safetensors(const struct dirent *d) {
    size_t n = strlen(d->d_name);
    return n > 12 && !strcmp(d->d_name + n - 12, ".safetensors");
}

int main(int argc, char **argv) {
    const int listing = argc == 3 && !strcmp(argv[1], "list");
    int mode = argc >= 4 ? (!strcmp(argv[1], "w8a16") ? 1 : !strcmp(argv[1], "w8a8") ? 2 : 0) : 0;
    if (!listing && (argc < 4 || argc > 5 || !mode)) {
        fprintf(stderr, "usage: %s w8a16|w8a8 TRANSFORMER_DIRECTORY CACHE_DIRECTORY [SCALE_GROUP]\n       %s list TRANSFORMER_DIRECTORY\n",
                argv[0], argv[0]);
        return 2;
    }
    char error[768] = {0};
    h3_gpu *gpu = NULL;
    int ok = 1;
    if (!listing) {
        setenv("H3_CUDA_WEIGHT_MODE", "stream", 1); /* nothing stays resident while preparing */
        gpu = h3_gpu_create("", error, sizeof error);
        if (!gpu) { fprintf(stderr, "h3q8_prepare: %s\n", error); return 1; }
        if (argc == 5) ok = h3q8_gpu_set_group(gpu, (uint32_t)strtoul(argv[4], NULL, 10));
        if (ok) ok = h3_gpu_quant_configure(gpu, mode, argv[3], 1 << 20, 1 << 20, 1);
        if (!ok) snprintf(error, sizeof error, "%s", h3_gpu_error(gpu));
    }
    struct dirent **files = NULL;
    int count = ok ? scandir(argv[2], &files, is_safetensors, by_name) : 0;
    unsigned done = 0;
    if (ok && count <= 0) { snprintf(error, sizeof error, "no .safetensors file in %s", argv[2]); ok = 0; }
    for (int i = 0; i < count; i++) {
        char *path = NULL;
        if (ok && asprintf(&path, "%s/%s", argv[2], files[i]->d_name) >= 0) {
            ok = prepare_file(gpu, path, &done, error, sizeof error);
            free(path);
        }
        free(files[i]);
    }
    free(files);
    if (ok && !done) { snprintf(error, sizeof error, "no DiT projection weight found in %s", argv[2]); ok = 0; }
    h3_gpu_stats stats;
    if (ok && gpu && h3_gpu_get_stats(gpu, &stats))
        fprintf(stderr, "h3q8_prepare: %u weights, %llu prepared, %llu already cached\n", done,
                (unsigned long long)stats.quant_cache_misses, (unsigned long long)stats.quant_cache_hits);
    if (!ok) fprintf(stderr, "h3q8_prepare: %s\n", error);
    h3_gpu_free(gpu);
    return ok ? 0 : 1;
}
