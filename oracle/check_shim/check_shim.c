/* Runtime of the check.h stand-in: suites are lists of (fixture, test) entries;
 * srunner_run_all runs them one by one - each in a forked child, as libcheck
 * does by default - and counts failures. */
#include <stdarg.h>
#include <stdlib.h>
#include <sys/wait.h>
#include <unistd.h>
#include "check.h"

#define MAX_TESTS 256
struct TCase {
  const char *name;
  SFun setup, teardown;
  TFun tests[MAX_TESTS];
  const char *names[MAX_TESTS];
  int n;
  struct TCase *next;
};
struct Suite {
  const char *name;
  TCase *first, *last;
};
struct SRunner {
  Suite *s;
  int failed, run;
  int nofork;
};

static jmp_buf escape;
static int in_test = 0, current_failed = 0;

Suite *suite_create(const char *name) {
  Suite *s = calloc(1, sizeof(*s));
  s->name = name;
  return s;
}
TCase *tcase_create(const char *name) {
  TCase *t = calloc(1, sizeof(*t));
  t->name = name;
  return t;
}
void tcase_set_timeout(TCase *tc, double seconds) { (void)tc; (void)seconds; }
void tcase_add_checked_fixture(TCase *tc, SFun setup, SFun teardown) {
  tc->setup = setup;
  tc->teardown = teardown;
}
void ga_shim_tcase_add_test(TCase *tc, TFun fn, const char *name) {
  if (tc->n < MAX_TESTS) {
    tc->tests[tc->n] = fn;
    tc->names[tc->n++] = name;
  }
}
void suite_add_tcase(Suite *s, TCase *tc) {
  if (s->last) s->last->next = tc;
  else s->first = tc;
  s->last = tc;
}
SRunner *srunner_create(Suite *s) {
  SRunner *r = calloc(1, sizeof(*r));
  r->s = s;
  return r;
}
void srunner_set_fork_status(SRunner *sr, enum fork_status st) { sr->nofork = st == CK_NOFORK; }

void ga_shim_fail(const char *file, int line, const char *fmt, ...) {
  va_list ap;
  fprintf(stdout, "  %s:%d: ", file, line);
  va_start(ap, fmt);
  vfprintf(stdout, fmt, ap);
  va_end(ap);
  fprintf(stdout, "\n");
  current_failed = 1;
  if (in_test) longjmp(escape, 1);
  exit(2);
}

void srunner_run_all(SRunner *sr, enum print_output mode) {
  TCase *tc;
  int i;
  (void)mode;
  printf("Running suite %s\n", sr->s->name);
  for (tc = sr->s->first; tc != NULL; tc = tc->next) {
    for (i = 0; i < tc->n; i++) {
      current_failed = 0;
      if (!sr->nofork) {
        /* like libcheck's default: every test in its own process */
        pid_t pid;
        int status = 0;
        fflush(stdout);
        pid = fork();
        if (pid == 0) {
          in_test = 1;
          if (setjmp(escape) == 0) {
            if (tc->setup) tc->setup();
            tc->tests[i](0);
            if (tc->teardown) tc->teardown();
          }
          fflush(stdout);
          _exit(current_failed ? 1 : 0);
        }
        if (pid < 0 || waitpid(pid, &status, 0) < 0 || !WIFEXITED(status) || WEXITSTATUS(status) != 0)
          current_failed = 1;
      } else {
        in_test = 1;
        if (setjmp(escape) == 0) {
          if (tc->setup) tc->setup();
          tc->tests[i](0);
          if (tc->teardown) tc->teardown();
        }
        in_test = 0;
      }
      sr->run++;
      sr->failed += current_failed;
      printf("%s:%s:%s: %s\n", sr->s->name, tc->name, tc->names[i], current_failed ? "FAILED" : "Passed");
      fflush(stdout);
    }
  }
  printf("%d%%: Checks: %d, Failures: %d\n", sr->run ? 100 * (sr->run - sr->failed) / sr->run : 100,
         sr->run, sr->failed);
}
int srunner_ntests_failed(SRunner *sr) { return sr->failed; }
void srunner_free(SRunner *sr) { free(sr); }
