/* Reader of the safetensors container the reference's checkpoints come in (its own reader: h3_safetensors.c;
 * the INT8-ConvRot DiT store on top of it: h3_dit_int8.c:120-206).  Layout of a file: 8 bytes little-endian header
 * length n, n bytes of JSON {"name": {"dtype": "I8", "shape": [..], "data_offsets": [begin, end]}, ...,
 * "__metadata__": {...}}, then the tensor data; offsets are relative to the end of the header.  The file is mapped
 * read-only; tensors are views into the mapping.  Plain C, no dependency. */
#define _GNU_SOURCE
#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "../../include/h3_b200.h"

struct h3b_ckpt {
    void *map;
    size_t map_bytes;
    const unsigned char *data;   /* first byte after the header */
    size_t data_bytes;
    h3b_ckpt_tensor *tensors;
    char **names;
    size_t count, cap;
};

static int fail(char *error, size_t error_size, const char *fmt, ...) {
    if (error && error_size) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(error, error_size, fmt, ap);
        va_end(ap);
    }
    return 0;
}

/* ---- a scanner for the subset of JSON a safetensors header uses */
typedef struct {
    const char *p, *end;
    const char *why;
} scan;

static void skip_ws(scan *s) {
    while (s->p < s->end && (*s->p == ' ' || *s->p == '\n' || *s->p == '\t' || *s->p == '\r')) s->p++;
}
static int expect(scan *s, char c) {
    skip_ws(s);
    if (s->p < s->end && *s->p == c) {
        s->p++;
        return 1;
    }
    s->why = "unexpected character";
    return 0;
}
/* string -> freshly allocated copy (escapes \" \\ \/ \n \t \r \b \f kept simple, \uXXXX copied verbatim) */
static char *scan_string(scan *s) {
    const char *q;
    char *out, *o;
    skip_ws(s);
    if (s->p >= s->end || *s->p != '"') {
        s->why = "string expected";
        return NULL;
    }
    q = ++s->p;
    while (q < s->end && *q != '"') q += (*q == '\\' && q + 1 < s->end) ? 2 : 1;
    if (q >= s->end) {
        s->why = "unterminated string";
        return NULL;
    }
    out = o = (char *)malloc((size_t)(q - s->p) + 1);
    if (!out) {
        s->why = "out of memory";
        return NULL;
    }
    while (s->p < q) {
        if (*s->p == '\\' && s->p + 1 < q) {
            char c = s->p[1];
            *o++ = c == 'n' ? '\n' : c == 't' ? '\t' : c == 'r' ? '\r' : c == 'b' ? '\b' : c == 'f' ? '\f' : c;
            s->p += 2;
        } else {
            *o++ = *s->p++;
        }
    }
    *o = 0;
    s->p = q + 1;
    return out;
}
static int scan_u64(scan *s, uint64_t *v) {
    uint64_t x = 0;
    int digits = 0;
    skip_ws(s);
    while (s->p < s->end && *s->p >= '0' && *s->p <= '9') {
        if (x > (UINT64_MAX - 9) / 10) {
            s->why = "number too large";
            return 0;
        }
        x = x * 10 + (uint64_t)(*s->p++ - '0');
        digits++;
    }
    if (!digits) {
        s->why = "non-negative integer expected";
        return 0;
    }
    *v = x;
    return 1;
}
/* skips any value (used for __metadata__ and unknown keys) */
static int skip_value(scan *s, int depth) {
    skip_ws(s);
    if (s->p >= s->end || depth > 32) {
        s->why = "value expected";
        return 0;
    }
    if (*s->p == '"') {
        char *t = scan_string(s);
        if (!t) return 0;
        free(t);
        return 1;
    }
    if (*s->p == '{' || *s->p == '[') {
        const char close = *s->p == '{' ? '}' : ']';
        const int is_obj = *s->p == '{';
        s->p++;
        skip_ws(s);
        if (s->p < s->end && *s->p == close) {
            s->p++;
            return 1;
        }
        for (;;) {
            if (is_obj) {
                char *k = scan_string(s);
                if (!k) return 0;
                free(k);
                if (!expect(s, ':')) return 0;
            }
            if (!skip_value(s, depth + 1)) return 0;
            skip_ws(s);
            if (s->p < s->end && *s->p == ',') {
                s->p++;
                continue;
            }
            return expect(s, close);
        }
    }
    /* number, true, false, null */
    while (s->p < s->end && *s->p != ',' && *s->p != '}' && *s->p != ']' && *s->p != ' ' && *s->p != '\n') s->p++;
    return 1;
}

static size_t dtype_bytes(const char *dt) {
    if (!strcmp(dt, "I8") || !strcmp(dt, "U8") || !strcmp(dt, "BOOL") || !strcmp(dt, "F8_E4M3") || !strcmp(dt, "F8_E5M2")) return 1;
    if (!strcmp(dt, "F16") || !strcmp(dt, "BF16") || !strcmp(dt, "I16") || !strcmp(dt, "U16")) return 2;
    if (!strcmp(dt, "F32") || !strcmp(dt, "I32") || !strcmp(dt, "U32")) return 4;
    if (!strcmp(dt, "F64") || !strcmp(dt, "I64") || !strcmp(dt, "U64")) return 8;
    return 0;
}

/* one tensor entry: {"dtype": "...", "shape": [...], "data_offsets": [b, e]} */
static int scan_entry(scan *s, h3b_ckpt_tensor *t, uint64_t *begin, uint64_t *end) {
    int have = 0;
    if (!expect(s, '{')) return 0;
    for (;;) {
        char *key = scan_string(s);
        if (!key) return 0;
        if (!expect(s, ':')) {
            free(key);
            return 0;
        }
        if (!strcmp(key, "dtype")) {
            char *v = scan_string(s);
            free(key);
            if (!v) return 0;
            snprintf(t->dtype, sizeof(t->dtype), "%s", v);
            free(v);
            have |= 1;
        } else if (!strcmp(key, "shape")) {
            free(key);
            if (!expect(s, '[')) return 0;
            t->rank = 0;
            skip_ws(s);
            if (s->p < s->end && *s->p == ']') {
                s->p++;
            } else {
                for (;;) {
                    uint64_t d;
                    if (!scan_u64(s, &d)) return 0;
                    if (t->rank >= 4) {
                        s->why = "tensor rank above 4";
                        return 0;
                    }
                    t->shape[t->rank++] = (size_t)d;
                    skip_ws(s);
                    if (s->p < s->end && *s->p == ',') {
                        s->p++;
                        continue;
                    }
                    if (!expect(s, ']')) return 0;
                    break;
                }
            }
            have |= 2;
        } else if (!strcmp(key, "data_offsets")) {
            free(key);
            if (!expect(s, '[') || !scan_u64(s, begin) || !expect(s, ',') || !scan_u64(s, end) || !expect(s, ']')) return 0;
            have |= 4;
        } else {
            free(key);
            if (!skip_value(s, 0)) return 0;
        }
        skip_ws(s);
        if (s->p < s->end && *s->p == ',') {
            s->p++;
            continue;
        }
        if (!expect(s, '}')) return 0;
        break;
    }
    if (have != 7) {
        s->why = "tensor entry lacks dtype, shape or data_offsets";
        return 0;
    }
    return 1;
}

void h3b_ckpt_close(h3b_ckpt *c) {
    size_t i;
    if (!c) return;
    for (i = 0; i < c->count; i++) free(c->names[i]);
    free(c->names);
    free(c->tensors);
    if (c->map && c->map != MAP_FAILED) munmap(c->map, c->map_bytes);
    free(c);
}

h3b_ckpt *h3b_ckpt_open(const char *path, char *error, size_t error_size) {
    struct stat st;
    h3b_ckpt *c;
    uint64_t hdr = 0;
    scan s;
    int fd, i;
    if (!path) {
        fail(error, error_size, "ckpt_open: NULL path");
        return NULL;
    }
    fd = open(path, O_RDONLY);
    if (fd < 0) {
        fail(error, error_size, "ckpt_open: %s: %s", path, strerror(errno));
        return NULL;
    }
    if (fstat(fd, &st) != 0 || st.st_size < 8) {
        close(fd);
        fail(error, error_size, "ckpt_open: %s: shorter than a safetensors header", path);
        return NULL;
    }
    c = (h3b_ckpt *)calloc(1, sizeof(*c));
    if (!c) {
        close(fd);
        fail(error, error_size, "ckpt_open: out of memory");
        return NULL;
    }
    c->map_bytes = (size_t)st.st_size;
    c->map = mmap(NULL, c->map_bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (c->map == MAP_FAILED) {
        fail(error, error_size, "ckpt_open: mmap(%s): %s", path, strerror(errno));
        c->map = NULL;
        h3b_ckpt_close(c);
        return NULL;
    }
    for (i = 7; i >= 0; i--) hdr = (hdr << 8) | ((const unsigned char *)c->map)[i];
    if (hdr > c->map_bytes - 8) {
        fail(error, error_size, "ckpt_open: %s: header length %llu exceeds the file", path, (unsigned long long)hdr);
        h3b_ckpt_close(c);
        return NULL;
    }
    c->data = (const unsigned char *)c->map + 8 + hdr;
    c->data_bytes = c->map_bytes - 8 - (size_t)hdr;
    s.p = (const char *)c->map + 8;
    s.end = s.p + hdr;
    s.why = NULL;
    if (!expect(&s, '{')) goto bad;
    skip_ws(&s);
    if (s.p < s.end && *s.p == '}') return c;   /* empty file */
    for (;;) {
        char *name = scan_string(&s);
        if (!name) goto bad;
        if (!expect(&s, ':')) {
            free(name);
            goto bad;
        }
        if (!strcmp(name, "__metadata__")) {
            free(name);
            if (!skip_value(&s, 0)) goto bad;
        } else {
            h3b_ckpt_tensor t;
            uint64_t b = 0, e = 0;
            size_t elems = 1, eb;
            int d;
            memset(&t, 0, sizeof(t));
            if (!scan_entry(&s, &t, &b, &e)) {
                free(name);
                goto bad;
            }
            eb = dtype_bytes(t.dtype);
            for (d = 0; d < t.rank; d++) elems *= t.shape[d];
            if (e < b || e > c->data_bytes || (eb && (e - b) != (uint64_t)elems * eb)) {
                fail(error, error_size, "ckpt_open: %s: tensor %s: offsets [%llu, %llu) do not fit its shape or the file", path,
                     name, (unsigned long long)b, (unsigned long long)e);
                free(name);
                h3b_ckpt_close(c);
                return NULL;
            }
            if (c->count == c->cap) {
                size_t ncap = c->cap ? 2 * c->cap : 64;
                h3b_ckpt_tensor *nt = (h3b_ckpt_tensor *)realloc(c->tensors, ncap * sizeof(*nt));
                char **nn = nt ? (char **)realloc(c->names, ncap * sizeof(*nn)) : NULL;
                if (nt) c->tensors = nt;
                if (nn) c->names = nn;
                if (!nt || !nn) {
                    free(name);
                    s.why = "out of memory";
                    goto bad;
                }
                c->cap = ncap;
            }
            t.data = c->data + b;
            t.bytes = (size_t)(e - b);
            t.name = name;
            c->names[c->count] = name;
            c->tensors[c->count++] = t;
        }
        skip_ws(&s);
        if (s.p < s.end && *s.p == ',') {
            s.p++;
            continue;
        }
        if (!expect(&s, '}')) goto bad;
        break;
    }
    return c;
bad:
    fail(error, error_size, "ckpt_open: %s: malformed header (%s at byte %ld)", path, s.why ? s.why : "?",
         (long)(s.p - ((const char *)c->map + 8)));
    h3b_ckpt_close(c);
    return NULL;
}

size_t h3b_ckpt_count(const h3b_ckpt *c) { return c ? c->count : 0; }

int h3b_ckpt_get(const h3b_ckpt *c, size_t index, h3b_ckpt_tensor *out) {
    if (!c || !out || index >= c->count) return 0;
    *out = c->tensors[index];
    return 1;
}

int h3b_ckpt_find(const h3b_ckpt *c, const char *name, h3b_ckpt_tensor *out) {
    size_t i;
    if (!c || !name) return 0;
    for (i = 0; i < c->count; i++)
        if (!strcmp(c->names[i], name)) {
            if (out) *out = c->tensors[i];
            return 1;
        }
    return 0;
}
