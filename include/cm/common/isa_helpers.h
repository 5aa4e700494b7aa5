/* Stand-in for the CM samples' common/isa_helpers.h as the reference's CM-flow drivers use it
 * (gemm-run-gpu-cm.cpp:30,73): there is no .isa file to load here, so loadFile returns the file's
 * name, which is what LoadProgram of this directory's cm_rt.h reads the design from. */
#ifndef T2SP_B200_CM_ISA_HELPERS_H
#define T2SP_B200_CM_ISA_HELPERS_H
#include <string>
namespace cm { namespace util { namespace isa {
inline std::string loadFile(const std::string &t2sp_name) { return t2sp_name; }
}}}
#endif
