/* Stand-in for dragon/utils/device/common_cuda.h: the host-only build of the
 * reference's converters needs nothing from it (TEST INFRASTRUCTURE ONLY). */
