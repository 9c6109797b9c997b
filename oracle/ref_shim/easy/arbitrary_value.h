// Stand-in for easy_profiler's macros (the reference sprinkles them through host code): all empty.
#pragma once
#define EASY_FUNCTION(...)
#define EASY_BLOCK(...)
#define EASY_END_BLOCK
#define EASY_VALUE(...)
#define EASY_PROFILER_ENABLE
