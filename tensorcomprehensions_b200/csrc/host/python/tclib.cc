// pybind11 module over the ATen-facing C++ API (the reference's tensor_comprehensions/pybinds/tclib.cc).
// Everything here goes through tc::aten::compile / run / profile / ATenAutotuner::tune; the extra
// introspection helpers (sexpr, analyze, match) exist for the CPU-side tests.
#include <torch/extension.h>

#include <sstream>

#include "tc/aten/aten_autotuner.h"
#include "tc/aten/aten_compiler.h"
#include "tc/core/flags.h"
#include "tc/lang/canonicalize.h"

namespace py = pybind11;
using tc::CudaBackend;
using tc::CudaMappingOptions;
using tc::CudaTcExecutor;

namespace {

std::vector<at::Tensor> metaInputs(const std::vector<std::vector<int64_t>>& shapes) {
  std::vector<at::Tensor> r;
  for (const auto& s : shapes) r.push_back(at::empty(s, at::TensorOptions().dtype(at::kFloat).device(at::kMeta)));
  return r;
}

// Shape-only descriptors (no data) for compile-time-only helpers.
std::vector<tc::DLConstTensorUPtr> shapeDescriptors(const std::vector<std::vector<int64_t>>& shapes,
                                                    const std::vector<std::string>& dtypes) {
  std::vector<tc::DLConstTensorUPtr> r;
  for (size_t i = 0; i < shapes.size(); ++i) {
    DLDataType dt{kDLFloat, 32, 1};
    if (i < dtypes.size()) {
      const std::string& d = dtypes[i];
      if (d == "float64" || d == "double") dt = DLDataType{kDLFloat, 64, 1};
      else if (d == "int32") dt = DLDataType{kDLInt, 32, 1};
      else if (d == "int64") dt = DLDataType{kDLInt, 64, 1};
      else if (d == "uint8") dt = DLDataType{kDLUInt, 8, 1};
    }
    r.push_back(tc::makeDLConstTensor(dt, DLDevice{kDLCUDA, 0}, shapes[i], tc::makeStridesFromSizes(shapes[i]), nullptr));
  }
  return r;
}

py::dict problemDict(const tc::MatchedLaunch& l) {
  py::dict d;
  const tcb200_problem_t& p = l.problem;
  d["family"] = l.family();
  d["epilogue"] = p.epilogue;
  d["accumulate"] = p.accumulate;
  d["inputs"] = l.inputs;
  d["output"] = l.output;
  d["statements"] = l.statements;
  if (p.family == TCB200_FAMILY_CONTRACTION) {
    d["batch"] = p.batch; d["M"] = p.M; d["N"] = p.N; d["K"] = p.K;
    d["a_k_major"] = p.a_k_major; d["b_k_major"] = p.b_k_major; d["bias_on_m"] = p.bias_on_m;
    d["lda"] = p.lda; d["ldb"] = p.ldb; d["ldc"] = p.ldc;
    d["stride_a"] = p.stride_a; d["stride_b"] = p.stride_b; d["stride_c"] = p.stride_c;
    d["batch_reduce"] = p.batch_reduce;
  } else if (p.family == TCB200_FAMILY_COPY) {
    d["elements"] = p.red[0];
  } else if (p.family == TCB200_FAMILY_REDUCTION) {
    d["red"] = std::vector<int64_t>(p.red, p.red + 3);
    d["reduce_op"] = p.reduce_op;
  } else if (p.family == TCB200_FAMILY_TENSORDOT) {
    d["td"] = std::vector<int64_t>(p.td, p.td + 5);
  } else {
    d["conv"] = std::vector<int64_t>(p.conv, p.conv + 8);
    d["conv_stride"] = std::vector<int64_t>{p.conv_stride[0] > 0 ? p.conv_stride[0] : 1, p.conv_stride[1] > 0 ? p.conv_stride[1] : 1};
  }
  return d;
}

tcb200_stream_t currentStream(const std::vector<at::Tensor>& inputs, py::object stream) {
  if (!stream.is_none()) return reinterpret_cast<tcb200_stream_t>(stream.cast<uintptr_t>());
  return nullptr;
}

struct PyExecutor {
  std::unique_ptr<CudaTcExecutor> exe;
  std::string tc, entry;
};

// The executor runs on the calling thread's current device (like the reference's); Python callers hand over
// tensors, so the device of the first input is made current for the duration of the call.
struct OnDeviceOf {
  explicit OnDeviceOf(const std::vector<at::Tensor>& inputs) {
    if (!inputs.empty() && inputs[0].is_cuda()) guard.reset(new tc::WithCudaDevice((size_t)inputs[0].get_device()));
  }
  std::unique_ptr<tc::WithCudaDevice> guard;
};

}  // namespace

PYBIND11_MODULE(tclib, m) {
  m.doc() = "Tensor Comprehensions on hand-written sm_100a kernels (C++ host bindings)";

  py::register_exception<lang::ErrorReport>(m, "ErrorReport");
  py::register_exception<tc::InvalidStrideException>(m, "InvalidStrideException");

  py::class_<CudaMappingOptions>(m, "MappingOptions")
      .def(py::init([](const std::string& preset) {
             if (preset == "naive") return CudaMappingOptions::makeNaiveMappingOptions();
             if (preset == "single_thread") return CudaMappingOptions::makeSingleThreadMappingOptions();
             if (preset == "pointwise") return CudaMappingOptions::makePointwiseMappingOptions();
             if (preset == "mlp") return CudaMappingOptions::makeMlpMappingOptions();
             if (preset == "conv") return CudaMappingOptions::makeConvolutionMappingOptions();
             if (preset == "group_conv") return CudaMappingOptions::makeGroupConvolutionMappingOptions();
             return CudaMappingOptions(preset);  // serialized form
           }),
           py::arg("preset") = "naive")
      .def("__str__", [](const CudaMappingOptions& o) { std::stringstream ss; ss << o; return ss.str(); })
      .def("__eq__", [](const CudaMappingOptions& a, const CudaMappingOptions& b) { return a == b; })
      // the bytes of a CudaMappingOptionsProto, as the reference's serialize() (tclib.cc:655-659);
      // the constructor takes them back (and this library's text form)
      .def("serialize", [](const CudaMappingOptions& o) { return py::bytes(o.toProtobufSerializedString()); })
      .def("serialize_text", &CudaMappingOptions::toSerializedString)
      .def("tile", [](CudaMappingOptions& o, const std::vector<uint64_t>& s) -> CudaMappingOptions& { return o.tile(s); }, py::return_value_policy::reference_internal)
      .def("unroll", [](CudaMappingOptions& o, uint64_t u) -> CudaMappingOptions& { return o.unroll(u); }, py::return_value_policy::reference_internal)
      .def("mapToThreads", [](CudaMappingOptions& o, const std::vector<uint64_t>& s) -> CudaMappingOptions& { return o.mapToThreads(s); }, py::return_value_policy::reference_internal)
      .def("mapToBlocks", [](CudaMappingOptions& o, const std::vector<uint64_t>& s) -> CudaMappingOptions& { return o.mapToBlocks(s); }, py::return_value_policy::reference_internal)
      .def("useSharedMemory", &CudaMappingOptions::useSharedMemory, py::return_value_policy::reference_internal)
      .def("usePrivateMemory", &CudaMappingOptions::usePrivateMemory, py::return_value_policy::reference_internal)
      .def("unrollCopyShared", &CudaMappingOptions::unrollCopyShared, py::return_value_policy::reference_internal)
      .def("useReadOnlyCache", &CudaMappingOptions::useReadOnlyCache, py::return_value_policy::reference_internal)
      .def("maxSharedMemory", &CudaMappingOptions::maxSharedMemory, py::return_value_policy::reference_internal)
      .def("matchLibraryCalls", [](CudaMappingOptions& o, bool b) -> CudaMappingOptions& { return o.matchLibraryCalls(b); }, py::return_value_policy::reference_internal)
      .def("fixParametersBeforeScheduling", [](CudaMappingOptions& o, bool b) -> CudaMappingOptions& { return o.fixParametersBeforeScheduling(b); }, py::return_value_policy::reference_internal)
      .def("scheduleFusionStrategy", [](CudaMappingOptions& o, const std::string& s) -> CudaMappingOptions& { return o.scheduleFusionStrategy(s); }, py::return_value_policy::reference_internal)
      .def("outerScheduleFusionStrategy", [](CudaMappingOptions& o, const std::string& s) -> CudaMappingOptions& { return o.outerScheduleFusionStrategy(s); }, py::return_value_policy::reference_internal)
      .def("intraTileScheduleFusionStrategy", [](CudaMappingOptions& o, const std::string& s) -> CudaMappingOptions& { return o.intraTileScheduleFusionStrategy(s); }, py::return_value_policy::reference_internal)
      .def_static("from_tile", [](int variant, int bm, int bn, int bk, int stages, int threads, int split, int split_k) {
        return CudaMappingOptions::fromTile(tcb200_tile_t{variant, bm, bn, bk, stages, threads, split, split_k});
      }, py::arg("variant"), py::arg("bm"), py::arg("bn"), py::arg("bk"), py::arg("stages"), py::arg("threads"),
         py::arg("split_tf32"), py::arg("split_k") = 0)
      .def("to_tile", [](const CudaMappingOptions& o) -> py::object {
        tcb200_tile_t t;
        if (!o.toTile(&t)) return py::none();
        return py::make_tuple(t.variant, t.bm, t.bn, t.bk, t.stages, t.threads, t.split_tf32, t.split_k);
      });

  py::class_<PyExecutor>(m, "TcExecutor")
      .def("run",
           [](PyExecutor& e, const std::vector<at::Tensor>& inputs, std::vector<at::Tensor> outputs, py::object stream) {
             if (outputs.empty()) outputs = tc::aten::prepareOutputs(e.tc, e.entry, inputs);
             auto in = tc::aten::makeDLConstTensors(inputs);
             auto out = tc::aten::makeDLTensors(outputs);
             OnDeviceOf dev(inputs);
             e.exe->run(tc::extractRawPtrs(in), tc::extractRawPtrs(out),
                        tc::CudaRuntimeInformation(currentStream(inputs, stream)));
             return outputs;
           },
           py::arg("inputs"), py::arg("outputs") = std::vector<at::Tensor>(), py::arg("stream") = py::none())
      .def("unchecked_run",
           [](PyExecutor& e, const std::vector<at::Tensor>& inputs, std::vector<at::Tensor> outputs, py::object stream) {
             std::vector<const void*> rawIn;
             std::vector<void*> rawOut;
             for (const auto& t : inputs) rawIn.push_back(t.data_ptr());
             for (auto& t : outputs) rawOut.push_back(t.data_ptr());
             OnDeviceOf dev(inputs);
             e.exe->uncheckedRun(rawIn, rawOut, tc::CudaRuntimeInformation(currentStream(inputs, stream)));
             return outputs;
           },
           py::arg("inputs"), py::arg("outputs"), py::arg("stream") = py::none())
      .def("profile",
           [](PyExecutor& e, const std::vector<at::Tensor>& inputs, std::vector<at::Tensor> outputs) {
             if (outputs.empty()) outputs = tc::aten::prepareOutputs(e.tc, e.entry, inputs);
             OnDeviceOf dev(inputs);
             tc::ProfilingInfo pi = tc::aten::profile(*e.exe, inputs, outputs);
             py::dict d;
             d["cpu_overhead_us"] = pi.cpuOverhead.toMicroSeconds();
             d["kernel_runtime_us"] = pi.kernelRuntimeUs;
             return d;
           },
           py::arg("inputs"), py::arg("outputs") = std::vector<at::Tensor>())
      .def("check_device_status",
           [](PyExecutor& e, int device, py::object stream) {
             tc::WithCudaDevice dev((size_t)device);
             e.exe->checkDeviceStatus(stream.is_none() ? nullptr : reinterpret_cast<tcb200_stream_t>(stream.cast<uintptr_t>()));
           },
           py::arg("device") = 0, py::arg("stream") = py::none(),
           "Waits for the stream and raises if a kernel's bounded device-side wait gave up since the last check.")
      .def_property_readonly("compiled_source", [](const PyExecutor& e) { return e.exe->compiledSource; })
      .def_property_readonly("num_launches", [](const PyExecutor& e) { return e.exe->numLaunches(); })
      .def_property_readonly("device", [](const PyExecutor& e) { return e.exe->device(); })
      .def_property_readonly("grid", [](const PyExecutor& e) { return e.exe->grid().extractVector(); })
      .def_property_readonly("block", [](const PyExecutor& e) { return e.exe->block().extractVector(); })
      .def("output_shapes", [](const PyExecutor& e) {
        std::vector<std::vector<int64_t>> r;
        for (const auto& i : e.exe->outputsInfo()) r.push_back(i.shape);
        return r;
      })
      .def("launches", [](const PyExecutor& e) {
        py::list r;
        for (const auto& l : e.exe->launches()) r.append(problemDict(l));
        return r;
      })
      .def("tiles", [](const PyExecutor& e) {
        py::list r;
        for (const auto& t : e.exe->tiles())
          r.append(py::make_tuple(t.variant, t.bm, t.bn, t.bk, t.stages, t.threads, t.split_tf32, t.split_k));
        return r;
      });

  m.def("compile",
        [](const std::string& tc, const std::string& entry, const std::vector<at::Tensor>& inputs,
           const CudaMappingOptions& options) {
          auto* e = new PyExecutor{tc::aten::compile<CudaBackend>(tc, entry, inputs, options), tc, entry};
          return std::unique_ptr<PyExecutor>(e);
        },
        py::arg("tc"), py::arg("entry_point"), py::arg("inputs"), py::arg("options"));

  m.def("prepare_outputs", [](const std::string& tc, const std::string& entry, const std::vector<at::Tensor>& inputs) {
    return tc::aten::prepareOutputs(tc, entry, inputs);
  });

  m.def("infer_output_shapes",
        [](const std::string& tc, const std::string& entry, const std::vector<std::vector<int64_t>>& shapes,
           const std::vector<std::string>& dtypes) {
          auto in = shapeDescriptors(shapes, dtypes);
          std::vector<std::vector<int64_t>> r;
          for (const auto& i : tc::inferOutputTensorInfo(tc, entry, tc::extractRawPtrs(in))) r.push_back(i.shape);
          return r;
        },
        py::arg("tc"), py::arg("entry_point"), py::arg("shapes"), py::arg("dtypes") = std::vector<std::string>());

  m.def("tune",
        [](const std::string& tc, const std::string& entry, const std::vector<at::Tensor>& inputs,
           const CudaMappingOptions& base, size_t topK) {
          tc::aten::ATenAutotuner<CudaBackend, tc::autotune::GeneticSearch> tuner(tc);
          return tuner.tune(entry, inputs, {base}, topK);
        },
        py::arg("tc"), py::arg("entry_point"), py::arg("inputs"), py::arg("base_options"), py::arg("top_k") = 1);

  // ---- options cache files (serialized CudaOptionsCacheProto, interchangeable with the reference's) ----
  // tensor_comprehensions/pybinds/tclib.cc:395-420: the k best options recorded for (tc, entry, sizes)
  m.def("cache_load",
        [](const std::string& filename, const std::string& tc, const std::string& entry,
           const std::vector<at::Tensor>& inputs, size_t count) {
          auto in = tc::aten::makeDLConstTensors(inputs);
          return tc::autotune::loadTopKFromCacheFile<CudaBackend>(tc, entry, filename, tc::extractRawPtrs(in), count);
        },
        py::arg("filename"), py::arg("tc"), py::arg("entry_point"), py::arg("inputs"), py::arg("count") = 1);
  // merges one (options, runtime) record into the file, keeping what it holds
  m.def("cache_store",
        [](const std::string& filename, const std::string& tc, const std::string& entry,
           const std::vector<at::Tensor>& inputs, const CudaMappingOptions& options, size_t runtimeUs) {
          auto in = tc::aten::makeDLConstTensors(inputs);
          auto raw = tc::extractRawPtrs(in);
          tc::autotune::OptionsCache<CudaBackend> cache;
          cache.loadCacheFromFile(filename);
          cache.recordRuntime(lang::canonicalTc(tc::detail::parse(tc).at(entry)), tc::makeTensorInfoVector(raw),
                              tc::inferOutputTensorInfo(tc, entry, raw), CudaBackend::backendString(), options,
                              tc::Duration::fromMicroSeconds(runtimeUs));
          cache.storeCacheToFile(filename);
        },
        py::arg("filename"), py::arg("tc"), py::arg("entry_point"), py::arg("inputs"), py::arg("options"),
        py::arg("runtime_us") = 0);
  m.def("cache_size", [](const std::string& filename) {
    tc::autotune::OptionsCache<CudaBackend> cache;
    cache.loadCacheFromFile(filename);
    return cache.size();
  });
  // tune and merge the best `top_k` of the sweep into `cache_filename` (the reference's Tuner with a
  // cache file: tclib.cc:570-580, options_cache-inl.h:353-367)
  m.def("tune_to_cache",
        [](const std::string& tc, const std::string& entry, const std::vector<at::Tensor>& inputs,
           const CudaMappingOptions& base, size_t topK, const std::string& cacheFilename) {
          tc::aten::ATenAutotuner<CudaBackend, tc::autotune::GeneticSearch> tuner(tc);
          auto best = tuner.tune(entry, inputs, {base}, topK);
          tc::autotune::appendTopKToCacheFile(*tuner.optionsCache, cacheFilename, (uint32_t)topK);
          return best;
        },
        py::arg("tc"), py::arg("entry_point"), py::arg("inputs"), py::arg("base_options"), py::arg("top_k"),
        py::arg("cache_filename"));

  m.def("tune_report",
        [](const std::string& tc, const std::string& entry, const std::vector<at::Tensor>& inputs) {
          std::vector<at::Tensor> outputs = tc::aten::prepareOutputs(tc, entry, inputs);
          auto in = tc::aten::makeDLConstTensors(inputs);
          auto out = tc::aten::makeDLTensors(outputs);
          py::list r;
          for (const auto& c : tc::autotune::sweepTiles(tc, entry, tc::extractRawPtrs(in), tc::extractRawPtrs(out), {}))
            r.append(py::make_tuple(c.options, c.medianUs, c.description));
          return r;
        });

  // ---- introspection for tests (no device needed) ---------------------------------------------
  m.def("sexpr", [](const std::string& tc, const std::string& mode) {
    std::stringstream out;
    lang::Parser parser(tc);
    while (parser.L.cur().kind != lang::TK_EOF) {
      auto def = parser.parseFunction();
      if (mode == "parse") {
        out << def;
      } else if (mode == "sema") {
        lang::Sema sema;
        auto checked = sema.checkFunction(def);
        out << checked << sema.dumpEnv();
      } else if (mode == "canon") {
        out << lang::canonicalize(lang::Sema().checkFunction(def));
      } else {
        throw std::runtime_error("unknown mode " + mode);
      }
    }
    return out.str();
  });
  m.def("parse_expr", [](const std::string& text) { std::stringstream out; out << lang::Parser(text).parseExp(); return out.str(); });
  m.def("parse_stmt", [](const std::string& text) { std::stringstream out; out << lang::Parser(text).parseStmt(); return out.str(); });
  m.def("canonical_tc", [](const std::string& tc) { return std::string(lang::canonicalTc(tc)); });

  m.def("analyze",
        [](const std::string& tc, const std::string& entry, const std::vector<std::vector<int64_t>>& shapes,
           const std::vector<std::string>& dtypes, bool throwWarnings) {
          auto in = shapeDescriptors(shapes, dtypes);
          tc::CompilerOptions opts;
          opts.throwWarnings = throwWarnings;
          opts.emitWarnings = false;
          auto parsed = tc::detail::parse(tc);
          auto it = parsed.find(entry);
          if (it == parsed.end()) throw std::runtime_error("undefined function " + entry);
          tc::DefAnalysis def = tc::analyzeDef(it->second, tc::extractRawPtrs(in), opts);
          py::dict d;
          d["sizes"] = def.sizes;
          py::list outs;
          for (const auto& o : def.outputs) outs.append(py::make_tuple(o.name, o.shape, lang::kindToString(o.scalarKind)));
          d["outputs"] = outs;
          py::list stmts;
          for (const auto& s : def.statements) {
            py::dict sd;
            sd["lhs"] = s.lhs;
            sd["indices"] = s.lhsIndices;
            sd["reduction"] = s.reductionVars;
            py::dict ranges;
            for (const auto& kv : s.ranges) ranges[py::str(kv.first)] = py::make_tuple(kv.second.min, kv.second.max + 1);
            sd["ranges"] = ranges;
            stmts.append(sd);
          }
          d["statements"] = stmts;
          return d;
        },
        py::arg("tc"), py::arg("entry_point"), py::arg("shapes"), py::arg("dtypes") = std::vector<std::string>(),
        py::arg("throw_warnings") = false);

  m.def("match",
        [](const std::string& tc, const std::string& entry, const std::vector<std::vector<int64_t>>& shapes) {
          auto in = shapeDescriptors(shapes, {});
          auto parsed = tc::detail::parse(tc);
          auto it = parsed.find(entry);
          if (it == parsed.end()) throw std::runtime_error("undefined function " + entry);
          tc::CompilerOptions opts;
          opts.emitWarnings = false;
          tc::DefAnalysis def = tc::analyzeDef(it->second, tc::extractRawPtrs(in), opts);
          py::list r;
          for (const auto& l : tc::matchKernels(def)) r.append(problemDict(l));
          return r;
        });

  m.def("set_flag", [](const std::string& name, const std::string& value) {
    std::string arg = "--" + name + "=" + value;
    char prog[] = "tclib";
    std::vector<char> buf(arg.begin(), arg.end());
    buf.push_back('\0');
    char* argv[] = {prog, buf.data()};
    if (tc::parseFlags(2, argv) != 1) throw std::runtime_error("unknown flag " + name);
  });
}
