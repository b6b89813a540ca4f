/* A minimal stand-in for libcheck's <check.h> (which is not installed here),
 * written for this repository: just enough of the API for the reference's C
 * test programs to compile UNMODIFIED from where they lie and run against this
 * library. Test infrastructure only. Each test runs in a forked child, in order; a
 * failed assertion prints its message and fails that test. */
#ifndef GA_CHECK_SHIM_H
#define GA_CHECK_SHIM_H

#include <setjmp.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define CHECK_MAJOR_VERSION 0
#define CHECK_MINOR_VERSION 15
#define CHECK_MICRO_VERSION 2

typedef struct Suite Suite;
typedef struct TCase TCase;
typedef struct SRunner SRunner;
typedef void (*TFun)(int);
typedef void (*SFun)(void);
enum print_output { CK_SILENT, CK_MINIMAL, CK_NORMAL, CK_VERBOSE };
enum fork_status { CK_FORK_GETENV, CK_FORK, CK_NOFORK };

Suite *suite_create(const char *name);
TCase *tcase_create(const char *name);
void tcase_set_timeout(TCase *tc, double seconds);
void tcase_add_checked_fixture(TCase *tc, SFun setup, SFun teardown);
void ga_shim_tcase_add_test(TCase *tc, TFun fn, const char *name);
#define tcase_add_test(tc, fn) ga_shim_tcase_add_test(tc, fn, #fn)
void suite_add_tcase(Suite *s, TCase *tc);
SRunner *srunner_create(Suite *s);
void srunner_set_fork_status(SRunner *sr, enum fork_status st);
void srunner_run_all(SRunner *sr, enum print_output mode);
int srunner_ntests_failed(SRunner *sr);
void srunner_free(SRunner *sr);

void ga_shim_fail(const char *file, int line, const char *fmt, ...)
    __attribute__((format(printf, 3, 4), noreturn));

#define START_TEST(name) static void name(int _i __attribute__((unused)))
#define END_TEST

#define ck_assert_msg(expr, ...) \
  do { if (!(expr)) ga_shim_fail(__FILE__, __LINE__, "Assertion '" #expr "' failed: " __VA_ARGS__); } while (0)
#define ck_assert(expr) ck_assert_msg(expr, " ")
#define ck_abort_msg(...) ga_shim_fail(__FILE__, __LINE__, __VA_ARGS__)

#define GA_SHIM_CMP(X, OP, Y, T, FMT)                                                       \
  do {                                                                                      \
    T ck_x_ = (T)(X);                                                                       \
    T ck_y_ = (T)(Y);                                                                       \
    if (!(ck_x_ OP ck_y_))                                                                  \
      ga_shim_fail(__FILE__, __LINE__, "Assertion '%s' failed: %s == " FMT ", %s == " FMT,  \
                   #X " " #OP " " #Y, #X, ck_x_, #Y, ck_y_);                                \
  } while (0)
#define ck_assert_int_eq(X, Y) GA_SHIM_CMP(X, ==, Y, intmax_t, "%jd")
#define ck_assert_int_ne(X, Y) GA_SHIM_CMP(X, !=, Y, intmax_t, "%jd")
#define ck_assert_uint_eq(X, Y) GA_SHIM_CMP(X, ==, Y, uintmax_t, "%ju")
#define ck_assert_uint_ne(X, Y) GA_SHIM_CMP(X, !=, Y, uintmax_t, "%ju")
#define ck_assert_ptr_eq(X, Y) GA_SHIM_CMP(X, ==, Y, const void *, "%p")
#define ck_assert_ptr_ne(X, Y) GA_SHIM_CMP(X, !=, Y, const void *, "%p")
#define ck_assert_float_eq(X, Y) GA_SHIM_CMP(X, ==, Y, float, "%g")
#define ck_assert_double_eq(X, Y) GA_SHIM_CMP(X, ==, Y, double, "%g")
#define ck_assert_str_eq(X, Y)                                                              \
  do {                                                                                      \
    const char *ck_x_ = (X), *ck_y_ = (Y);                                                  \
    if (ck_x_ == NULL || ck_y_ == NULL || strcmp(ck_x_, ck_y_) != 0)                        \
      ga_shim_fail(__FILE__, __LINE__, "Assertion '%s' failed: \"%s\" vs \"%s\"",           \
                   #X " == " #Y, ck_x_ ? ck_x_ : "(null)", ck_y_ ? ck_y_ : "(null)");       \
  } while (0)

#endif
