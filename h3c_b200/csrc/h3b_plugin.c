/* Exported view of the switch registry (include/h3b_plugin.h) for callers that cannot include a C header:
 * the Python harness and the bench read their switches through these, so that every read goes through the
 * catalogue. */
#include "../../include/h3_b200.h"
#include "../../include/h3b_plugin.h"

size_t h3b_plugin_count(void) { return h3_plugin_builtin_count; }

int h3b_plugin_get(size_t index, const char **name, const char **status, const char **stage, const char **default_value) {
    if (index >= h3_plugin_builtin_count) return 0;
    if (name) *name = h3_plugin_builtins[index].name;
    if (status) *status = h3_plugin_builtins[index].status;
    if (stage) *stage = h3_plugin_builtins[index].stage;
    if (default_value) *default_value = h3_plugin_builtins[index].default_value;
    return 1;
}

const char *h3b_plugin_value(const char *name) { return h3_plugin_value(name); }

int h3b_plugin_enabled(const char *name) { return h3_plugin_enabled(name); }
