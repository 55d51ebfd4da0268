// spconv::load_engine_from_onnx for the v1.3 interface, exported by libspconv.so.
// Same signature as the loader the reference compiles into each application from
// libraries/3DSparseConvolution/src/onnx-parser.hpp:32-40; this one reads the protobuf
// wire format itself, so neither libprotobuf nor the generated onnx-ml.pb.* files are needed.
#ifndef ONNX_PARSER_HPP
#define ONNX_PARSER_HPP

#include <spconv/engine.hpp>

namespace spconv {

Exported std::shared_ptr<Engine> load_engine_from_onnx(
    const std::string& onnx_file,
    Precision inference_precision = Precision::Float16,  // Float16 overrides per-layer precisions
    bool sortmask = false,                                // ignored
    bool enable_blackwell = false,                        // ignored: always on
    bool with_auxiliary_stream = false,                   // ignored
    unsigned int fixed_launch_points = 10000,             // launch-size hint (CUDA graph / DDS)
    void* stream = nullptr);                              // stream used for the weight upload

}  // namespace spconv

#endif  // ONNX_PARSER_HPP
