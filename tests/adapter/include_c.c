/* A plain-C translation unit that includes the boundary header and names every
 * entry point through a function pointer of its declared type: the header must be
 * valid C99 (no C++ in it) and the library must export what it declares. */
#include <stdio.h>

#include "b2vm.h"

int main(void) {
  b2_status (*create)(int, b2_runtime **, char *, size_t) = b2_runtime_create;
  b2_status (*parse)(const uint8_t *, size_t, b2_program **, char *, size_t) = b2_program_parse;
  b2_status (*load)(b2_runtime *, b2_program *, b2_loaded **, char *, size_t) = b2_program_load;
  b2_status (*exec_host)(b2_loaded *, const void *const *, size_t, void *const *, size_t, char *, size_t) = b2_execute_host;
  b2_status (*exec_dev)(b2_loaded *, void *const *, size_t, void **, size_t, char *, size_t) = b2_execute_device;
  int (*in_out)(const b2_loaded *, uint32_t) = b2_loaded_in_out_result;
  /* host-only calls: a garbage blob is refused by the parser, no device needed */
  static const uint8_t junk[64] = {1, 2, 3};
  b2_program *p = NULL;
  char err[256];
  const b2_status st = parse(junk, sizeof junk, &p, err, sizeof err);
  printf("parse(junk) -> %d (%s); static sum capacity %llu floats\n", (int)st, err,
         (unsigned long long)b2_sum_f32_static_max_elems());
  return (st == B2_INVALID_ARGUMENT && p == NULL && create && load && exec_host && exec_dev && in_out) ? 0 : 1;
}
