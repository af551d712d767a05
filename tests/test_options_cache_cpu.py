"""The options-cache file and the serialized mapping options are protocol-buffers messages of the
reference's schema (tc/proto/mapping_options.proto:19-91, tc/proto/compcache.proto:19-62), written and
parsed here without a protobuf library.  The Python protobuf runtime, given that schema, is the second
implementation: it must read what this library writes, and this library must read what it writes."""
import pytest
import torch

import tensorcomprehensions_b200 as tc
from tensorcomprehensions_b200 import tclib
from tensorcomprehensions_b200 import workloads as wl

pb = pytest.importorskip("google.protobuf")
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory  # noqa: E402

F = descriptor_pb2.FieldDescriptorProto
REQ, OPT, REP = F.LABEL_REQUIRED, F.LABEL_OPTIONAL, F.LABEL_REPEATED
U64, U32, BOOL, STR, MSG, ENUM = F.TYPE_UINT64, F.TYPE_UINT32, F.TYPE_BOOL, F.TYPE_STRING, F.TYPE_MESSAGE, F.TYPE_ENUM

# message -> [(field, number, label, type, type name)]: the schema as the two .proto files give it
SCHEMA = {
    "CudaDimProto": [("x", 1, REQ, U64, None), ("y", 2, OPT, U64, None), ("z", 3, OPT, U64, None)],
    "SchedulerOptionsProto": [("fusion_strategy", 1, REQ, ENUM, ".tc.FusionStrategy"),
                              ("allow_skewing", 2, REQ, BOOL, None), ("positive_orthant", 3, REQ, BOOL, None)],
    "TilingProto": [("sizes", 1, REP, U64, None)],
    "MappingOptionsProto": [("outer_schedule_options", 1, REQ, MSG, ".tc.SchedulerOptionsProto"),
                            ("intra_tile_schedule_options", 2, REQ, MSG, ".tc.SchedulerOptionsProto"),
                            ("fix_parameters_before_scheduling", 3, REQ, BOOL, None),
                            ("tiling", 4, OPT, MSG, ".tc.TilingProto"), ("unroll", 5, OPT, U64, None),
                            ("tile_imperfectly_nested", 6, REQ, BOOL, None),
                            ("match_library_calls", 7, REQ, BOOL, None)],
    "CudaMappingOptionsProto": [("generic_mapping_options", 1, REQ, MSG, ".tc.MappingOptionsProto"),
                                ("block", 2, REQ, MSG, ".tc.CudaDimProto"), ("grid", 3, REQ, MSG, ".tc.CudaDimProto"),
                                ("use_shared_memory", 4, REQ, BOOL, None), ("use_private_memory", 5, REQ, BOOL, None),
                                ("unroll_copy_shared", 6, REQ, BOOL, None), ("max_shared_memory", 7, OPT, U64, None),
                                ("use_readonly_cache", 8, REQ, BOOL, None), ("private_depth", 9, OPT, U32, None),
                                ("shared_depth", 10, OPT, U32, None)],
    "DLDataTypeProto": [("code", 1, REQ, U32, None), ("bits", 2, REQ, U32, None), ("lanes", 3, REQ, U32, None)],
    "TensorInfoProto": [("shape", 1, REP, U64, None), ("strides", 2, REP, U64, None), ("alignment", 3, REQ, U64, None),
                        ("dtype", 4, REQ, MSG, ".tc.DLDataTypeProto")],
    "OptionsCacheKeyProto": [("id", 1, REQ, STR, None), ("inputs", 2, REP, MSG, ".tc.TensorInfoProto"),
                             ("outputs", 3, REP, MSG, ".tc.TensorInfoProto"), ("backend_str", 4, REQ, STR, None),
                             ("git_version", 5, REQ, STR, None)],
    "CudaOptionsCacheValueProto": [("kernel_options", 1, REQ, MSG, ".tc.CudaMappingOptionsProto"),
                                   ("recorded_runtimes", 2, REP, U64, None)],
    "CudaOptionsCacheProto": [("keys", 1, REP, MSG, ".tc.OptionsCacheKeyProto"),
                              ("values", 2, REP, MSG, ".tc.CudaOptionsCacheValueProto")],
}


@pytest.fixture(scope="module")
def msgs():
    fdp = descriptor_pb2.FileDescriptorProto(name="tc_cache_schema.proto", package="tc", syntax="proto2")
    e = fdp.enum_type.add(name="FusionStrategy")
    for name, number in (("Max", 1), ("Preserve3Coincident", 2), ("Min", 3)):
        e.value.add(name=name, number=number)
    for mname, fields in SCHEMA.items():
        m = fdp.message_type.add(name=mname)
        for fname, number, label, ftype, tname in fields:
            f = m.field.add(name=fname, number=number, label=label, type=ftype)
            if tname:
                f.type_name = tname
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fdp)
    return {n: message_factory.GetMessageClass(pool.FindMessageTypeByName("tc." + n)) for n in SCHEMA}


def test_mapping_options_bytes_parse_as_the_reference_proto(msgs):
    o = tc.MappingOptions("naive")
    o.tile([4, 8, 16]).unroll(64).mapToThreads([32, 4]).mapToBlocks([100, 7, 3]).useSharedMemory(True)
    o.maxSharedMemory(40000).scheduleFusionStrategy("Max").matchLibraryCalls(True).useReadOnlyCache(True)
    p = msgs["CudaMappingOptionsProto"]()
    p.ParseFromString(o.serialize())
    assert p.IsInitialized()  # every required field of the schema is on the wire
    g = p.generic_mapping_options
    assert list(g.tiling.sizes) == [4, 8, 16] and g.unroll == 64 and g.match_library_calls
    assert g.outer_schedule_options.fusion_strategy == 1 and g.intra_tile_schedule_options.fusion_strategy == 1
    assert g.outer_schedule_options.positive_orthant and not g.outer_schedule_options.allow_skewing
    assert (p.block.x, p.block.y, p.block.HasField("z")) == (32, 4, False)
    assert (p.grid.x, p.grid.y, p.grid.z) == (100, 7, 3)
    assert p.use_shared_memory and not p.use_private_memory and p.use_readonly_cache
    assert p.max_shared_memory == 40000
    # and back: bytes produced by the protobuf runtime (packed or not) load here
    p.generic_mapping_options.tiling.sizes[:] = [5, 6]
    p.block.z = 2
    back = tc.MappingOptions(p.SerializeToString())
    q = msgs["CudaMappingOptionsProto"]()
    q.ParseFromString(back.serialize())
    assert q == p
    assert tc.MappingOptions(o.serialize()) == o and tc.MappingOptions(o.serialize_text()) == o


def test_tile_encoding_survives_the_proto(msgs):
    o = tc.MappingOptions.from_tile(5, 256, 128, 32, 8, 608, 3)
    p = msgs["CudaMappingOptionsProto"]()
    p.ParseFromString(o.serialize())
    assert (p.private_depth, p.shared_depth) == (5, 3) and list(p.generic_mapping_options.tiling.sizes) == [256, 128, 32]
    assert tc.MappingOptions(p.SerializeToString()).to_tile() == (5, 256, 128, 32, 8, 608, 3, 0)


def test_cache_file_is_a_cuda_options_cache_proto(tmp_path, msgs):
    path = str(tmp_path / "cache.cuda.options")
    cache = tc.MappingOptionsCache(path)
    ins = [torch.empty(4, 6), torch.empty(5, 6)]
    fast, slow = tc.MappingOptions.from_tile(1, 64, 64, 16, 0, 256, 0), tc.MappingOptions.from_tile(1, 32, 32, 16, 0, 128, 0)
    cache.store(wl.TMM_TC, "tmm", ins, slow, runtime_us=90)
    cache.store(wl.TMM_TC, "tmm", ins, fast, runtime_us=30)
    cache.store(wl.TMM_TC, "tmm", ins, fast, runtime_us=34)
    p = msgs["CudaOptionsCacheProto"]()
    p.ParseFromString(open(path, "rb").read())
    assert p.IsInitialized() and len(p.keys) == len(p.values) == 2
    k = p.keys[0]
    assert k.id == tclib.canonical_tc(wl.TMM_TC) and p.keys[1] == k
    assert [list(t.shape) for t in k.inputs] == [[4, 6], [5, 6]] and [list(t.strides) for t in k.inputs] == [[6, 1], [6, 1]]
    assert [list(t.shape) for t in k.outputs] == [[4, 5]]
    assert (k.inputs[0].dtype.code, k.inputs[0].dtype.bits, k.inputs[0].dtype.lanes) == (2, 32, 1)  # kDLFloat
    runtimes = sorted(sorted(v.recorded_runtimes) for v in p.values)
    assert runtimes == [[30, 34], [90]]

    # a file written by the protobuf runtime: one more, faster candidate for the same key, its
    # runtimes packed, plus an entry of another revision that must not be returned
    best = tc.MappingOptions.from_tile(1, 64, 32, 16, 0, 256, 0)
    v = p.values.add()
    v.kernel_options.ParseFromString(best.serialize())
    v.recorded_runtimes.extend([11, 12, 13])
    p.keys.add().CopyFrom(k)
    other = p.keys.add()
    other.CopyFrom(k)
    other.git_version = "0123abc"
    w = p.values.add()
    w.kernel_options.ParseFromString(slow.serialize())
    w.recorded_runtimes.append(1)
    path2 = str(tmp_path / "from_protobuf.options")
    open(path2, "wb").write(p.SerializeToString())
    got = tc.MappingOptionsCache(path2).load(wl.TMM_TC, "tmm", ins, 10)
    assert got == [best, fast, slow]
    assert len(tc.MappingOptionsCache(path2)) == 4


def test_malformed_cache_is_an_error(tmp_path):
    path = str(tmp_path / "bad.options")
    open(path, "wb").write(b"\x0a\xff\xff\xff")  # a length that runs past the end of the file
    with pytest.raises(RuntimeError, match="options cache"):
        tc.MappingOptionsCache(path).load(wl.TMM_TC, "tmm", [torch.empty(4, 6), torch.empty(5, 6)])
    with pytest.raises(RuntimeError, match="CudaMappingOptionsProto"):
        tc.MappingOptions(b"\x08\x01")
