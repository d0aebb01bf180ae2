/* Thread-local sticky error state: code + message, cleared only on request
 * (same contract as the reference's Src/Spingalett.Error.c:9-28; its loader
 * relies on the stickiness, Serialize.c:556). */
#include "spg_internal.h"
#include <stdarg.h>
#include <stdio.h>

static _Thread_local int  t_code = SPINGALETT_OK;
static _Thread_local char t_msg[SPG_ERRMSG_MAX];

int spingalett_last_error_code(void) { return t_code; }
const char *spingalett_last_error_message(void) { return t_msg; }
void spingalett_clear_error(void) { t_code = SPINGALETT_OK; t_msg[0] = 0; }

void spg_set_error(int code, const char *msg)
{
    t_code = code;
    snprintf(t_msg, sizeof t_msg, "%s", msg ? msg : "unknown error");
}

void spg_set_errorf(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    t_code = code;
    vsnprintf(t_msg, sizeof t_msg, fmt, ap);
    va_end(ap);
}
