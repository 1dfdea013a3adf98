/* Compiled by tests/test_struct_layout.py with the reference's zfp directory on
 * the include path: every size and member offset of the zfp objects the
 * compatibility header mirrors must equal the reference's own
 * (CSWAP+/zfp/zfp.h:95-102,140-145 and struct bitstream, bitstream.c:131-141,
 * which is included as source because the struct is private to that file). */
#include <stddef.h>
#include <stdint.h>

#include "zfp.h"
#define inline_
#include "bitstream.c"

#include "cswap_compat.h"

#define SAME_SIZE(a, b) _Static_assert(sizeof(a) == sizeof(b), "size of " #a)
#define SAME_OFF(a, b, m) _Static_assert(offsetof(a, m) == offsetof(b, m), "offset of " #a "." #m)

SAME_SIZE(zfp_stream, csw_zfp_stream);
SAME_OFF(zfp_stream, csw_zfp_stream, minbits);
SAME_OFF(zfp_stream, csw_zfp_stream, maxbits);
SAME_OFF(zfp_stream, csw_zfp_stream, maxprec);
SAME_OFF(zfp_stream, csw_zfp_stream, minexp);
SAME_OFF(zfp_stream, csw_zfp_stream, stream);
SAME_OFF(zfp_stream, csw_zfp_stream, exec);

SAME_SIZE(zfp_field, csw_zfp_field);
SAME_OFF(zfp_field, csw_zfp_field, type);
SAME_OFF(zfp_field, csw_zfp_field, nx);
SAME_OFF(zfp_field, csw_zfp_field, ny);
SAME_OFF(zfp_field, csw_zfp_field, nz);
SAME_OFF(zfp_field, csw_zfp_field, nw);
SAME_OFF(zfp_field, csw_zfp_field, sx);
SAME_OFF(zfp_field, csw_zfp_field, sy);
SAME_OFF(zfp_field, csw_zfp_field, sz);
SAME_OFF(zfp_field, csw_zfp_field, sw);
SAME_OFF(zfp_field, csw_zfp_field, data);

SAME_SIZE(struct bitstream, csw_bitstream);
SAME_OFF(struct bitstream, csw_bitstream, bits);
SAME_OFF(struct bitstream, csw_bitstream, buffer);
SAME_OFF(struct bitstream, csw_bitstream, ptr);
SAME_OFF(struct bitstream, csw_bitstream, begin);
SAME_OFF(struct bitstream, csw_bitstream, end);

_Static_assert(zfp_type_float == 3, "zfp_type_float");
_Static_assert(sizeof(word) == 8, "64-bit stream words");

int layout_check_ok(void) { return 1; }
