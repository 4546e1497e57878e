/* Empty stand-in for <gtest/gtest.h>: the reference's test/test.hpp includes it but the two
 * functions taken from that header (init_matrix, sgemm_cpu) use nothing from GoogleTest. */
#ifndef ORACLE_SHIM_GTEST_H
#define ORACLE_SHIM_GTEST_H
#endif
