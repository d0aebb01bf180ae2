/*
 * Drop-in include path for programs written against pka-human/Spingalett:
 * `#include <Spingalett/Spingalett.h>` keeps compiling unchanged.  All
 * declarations live in spingalett_b200.h.
 */
#pragma once
#include "Spingalett.Config.h"
#include "../spingalett_b200.h"
