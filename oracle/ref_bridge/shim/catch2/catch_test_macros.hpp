// Stand-in for Catch2's macro header, used ONLY to compile the reference
// project's end-to-end test translation units into the checker library under
// oracle/_ref. The test bodies are never run: each TEST_CASE becomes a function
// template that is never instantiated, so only the free helper functions of
// those files (input generators and fp64 references) end up in the library.
#pragma once
#define KHREF_CAT2(a, b) a##b
#define KHREF_CAT(a, b) KHREF_CAT2(a, b)
#define TEST_CASE(...) \
  template <int KhrefUnused> static void KHREF_CAT(khref_test_case_, __LINE__)()
#define REQUIRE(...) ((void)sizeof((__VA_ARGS__) ? 1 : 0))
#define REQUIRE_FALSE(...) ((void)sizeof((__VA_ARGS__) ? 1 : 0))
#define CHECK(...) ((void)sizeof((__VA_ARGS__) ? 1 : 0))
#define CHECK_FALSE(...) ((void)sizeof((__VA_ARGS__) ? 1 : 0))
#define SKIP(...) return
#define FAIL(...) ((void)0)
#define INFO(...) ((void)0)
#define SUCCEED(...) ((void)0)
