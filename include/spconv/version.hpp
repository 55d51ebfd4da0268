// Interface generation this library implements: the reference's v1.3.2 headers
// (libraries/3DSparseConvolution/libspconv/include/spconv/version.hpp:16-18).
// NVSPCONV_VERSION is the string callers print, e.g. "1.3.2".
#ifndef __SPCONV_VERSION_HPP__
#define __SPCONV_VERSION_HPP__

#define NVSPCONV_MAJOR 1
#define NVSPCONV_MINOR 3
#define NVSPCONV_REL 2

#define NVSPCONV_STR_(v) #v
#define NVSPCONV_STR(v) NVSPCONV_STR_(v)
#define NVSPCONV_VERSION NVSPCONV_STR(NVSPCONV_MAJOR) "." NVSPCONV_STR(NVSPCONV_MINOR) "." NVSPCONV_STR(NVSPCONV_REL)
#define NVSPCONV_BACKEND "b200 (sm_100a)"

#endif  // __SPCONV_VERSION_HPP__
