"""Checkpoint interchange (deepnet/util.py:13-53, deepnet/protos/deepnet.proto): the hand-written
wire codec against the protobuf runtime on descriptors restating the reference's field numbers."""
import gzip
import os

import numpy as np
import pytest

from deepnet_b200 import checkpoint as ck


def reference_messages():
    """Message classes for the subset of deepnet.proto the checkpoints use, built at run time
    (field numbers and types as in deepnet/protos/deepnet.proto:7-50,181-229,231-257)."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    T = descriptor_pb2.FieldDescriptorProto
    fd = descriptor_pb2.FileDescriptorProto(name="deepnet_subset.proto", package="deepnet", syntax="proto2")

    def msg(name, fields):
        m = fd.message_type.add(name=name)
        for fname, num, ftype, label, tname in fields:
            f = m.field.add(name=fname, number=num, type=ftype, label=label)
            if tname:
                f.type_name = ".deepnet." + tname
    OPT, REQ, REP = T.LABEL_OPTIONAL, T.LABEL_REQUIRED, T.LABEL_REPEATED
    msg("Parameter", [("name", 1, T.TYPE_STRING, REQ, None), ("mat", 2, T.TYPE_BYTES, OPT, None),
                      ("dimensions", 3, T.TYPE_INT32, REP, None), ("initialization", 4, T.TYPE_INT32, OPT, None),
                      ("sigma", 5, T.TYPE_FLOAT, OPT, None)])
    msg("Hyperparams", [("base_epsilon", 1, T.TYPE_FLOAT, OPT, None)])
    msg("Layer", [("name", 1, T.TYPE_STRING, REQ, None), ("dimensions", 3, T.TYPE_INT32, REQ, None),
                  ("param", 5, T.TYPE_MESSAGE, REP, "Parameter"), ("is_input", 7, T.TYPE_BOOL, OPT, None),
                  ("hyperparams", 10, T.TYPE_MESSAGE, OPT, "Hyperparams"), ("loss_weight", 19, T.TYPE_FLOAT, OPT, None)])
    msg("Edge", [("node1", 1, T.TYPE_STRING, REQ, None), ("node2", 2, T.TYPE_STRING, REQ, None),
                 ("directed", 3, T.TYPE_BOOL, OPT, None), ("param", 4, T.TYPE_MESSAGE, REP, "Parameter"),
                 ("up_factor", 9, T.TYPE_FLOAT, OPT, None)])
    msg("Model", [("name", 1, T.TYPE_STRING, REQ, None), ("model_type", 2, T.TYPE_INT32, REQ, None),
                  ("layer", 3, T.TYPE_MESSAGE, REP, "Layer"), ("edge", 4, T.TYPE_MESSAGE, REP, "Edge"),
                  ("seed", 9, T.TYPE_INT32, OPT, None), ("positive_phase_order", 10, T.TYPE_STRING, REP, None)])
    msg("Operation", [("optimizer", 1, T.TYPE_INT32, REQ, None), ("current_step", 4, T.TYPE_INT32, OPT, None),
                      ("batchsize", 5, T.TYPE_INT32, OPT, None)])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = getattr(message_factory, "GetMessageClass", None)
    if get is None:
        factory = message_factory.MessageFactory(pool)
        get = factory.GetPrototype
    return {n: get(pool.FindMessageTypeByName("deepnet." + n)) for n in
            ("Parameter", "Layer", "Edge", "Model", "Operation")}


def test_varints_and_negative_int32():
    fields = [(1, ck.VARINT, 0), (2, ck.VARINT, 300), (3, ck.VARINT, -1), (4, ck.BYTES, b"abc"),
              (5, ck.FIXED32, b"\x00\x00\x80\x3f")]
    out = ck.decode(ck.encode(fields))
    assert out[0][2] == 0 and out[1][2] == 300 and ck._signed32(out[2][2]) == -1 and out[3][2] == b"abc"
    assert out[4][2] == b"\x00\x00\x80\x3f"


def test_model_written_here_parses_with_the_protobuf_runtime():
    M = reference_messages()
    rng = np.random.default_rng(0)
    w = rng.standard_normal((7, 5)).astype(np.float32)
    bv, bh = rng.standard_normal(7).astype(np.float32), rng.standard_normal(5).astype(np.float32)
    m = ck.Model("rbm1", ck.MODEL_DBM)
    m.add_layer("input_layer", 7, bias=bv, is_input=True)
    m.add_layer("hidden1", 5, bias=bh)
    m.add_edge("input_layer", "hidden1", w)
    ref = M["Model"]()
    ref.ParseFromString(m.to_bytes())
    assert ref.name == "rbm1" and ref.model_type == 3
    assert [l.name for l in ref.layer] == ["input_layer", "hidden1"] and ref.layer[0].is_input
    assert ref.layer[0].dimensions == 7 and list(ref.layer[0].param[0].dimensions) == [7, 1]
    got_w = np.frombuffer(ref.edge[0].param[0].mat, dtype=np.float32).reshape(*ref.edge[0].param[0].dimensions)
    np.testing.assert_array_equal(got_w, w)       # deepnet/util.py:13-16
    np.testing.assert_array_equal(np.frombuffer(ref.layer[1].param[0].mat, np.float32), bh)


def test_model_written_by_the_protobuf_runtime_round_trips_with_unknown_fields_kept():
    M = reference_messages()
    rng = np.random.default_rng(1)
    w = rng.standard_normal((6, 4)).astype(np.float32)
    ref = M["Model"](name="m", model_type=3, seed=42)
    ref.positive_phase_order.extend(["a", "b"])
    la = ref.layer.add(name="v", dimensions=6, is_input=True, loss_weight=0.5)
    la.hyperparams.base_epsilon = 0.125
    p = la.param.add(name="bias", mat=np.zeros(6, np.float32).tobytes(), initialization=2, sigma=0.25)
    p.dimensions.extend([6, 1])
    lb = ref.layer.add(name="h", dimensions=4)
    pb = lb.param.add(name="bias", mat=np.ones(4, np.float32).tobytes())
    pb.dimensions.extend([4, 1])
    e = ref.edge.add(node1="v", node2="h", directed=False, up_factor=2.0)
    pw = e.param.add(name="weight", mat=w.tobytes())
    pw.dimensions.extend([6, 4])
    m = ck.Model.from_bytes(ref.SerializeToString())
    assert m.name == "m" and m.layer_names() == ["v", "h"] and m.edge_names() == [("v", "h")]
    assert m.layer_dimensions("h") == 4
    np.testing.assert_array_equal(m.get_edge_param("v", "h"), w)
    np.testing.assert_array_equal(m.get_layer_param("h"), np.ones((4, 1), np.float32))
    # modify the weight and one bias; everything this module does not interpret must survive
    m.set_edge_param("v", "h", w * 2)
    m.set_layer_param("v", np.full((6, 1), 3.0, np.float32))
    back = M["Model"]()
    back.ParseFromString(m.to_bytes())
    assert back.seed == 42 and list(back.positive_phase_order) == ["a", "b"]
    assert back.layer[0].hyperparams.base_epsilon == 0.125 and back.layer[0].loss_weight == 0.5
    assert back.layer[0].param[0].initialization == 2 and back.layer[0].param[0].sigma == 0.25
    assert back.edge[0].up_factor == 2.0 and back.edge[0].directed is False
    np.testing.assert_array_equal(np.frombuffer(back.edge[0].param[0].mat, np.float32).reshape(6, 4), w * 2)
    np.testing.assert_array_equal(np.frombuffer(back.layer[0].param[0].mat, np.float32), np.full(6, 3.0, np.float32))


def test_checkpoint_files_and_resume_step(tmp_path):
    M = reference_messages()
    m = ck.Model("net", ck.MODEL_DBM)
    m.add_layer("v", 3, bias=np.zeros(3))
    m.add_layer("h", 2, bias=np.zeros(2))
    m.add_edge("v", "h", np.arange(6, dtype=np.float32).reshape(3, 2))
    op = M["Operation"](optimizer=4, current_step=0, batchsize=100).SerializeToString()
    op = ck.operation_with_step(op, 1234)
    last = ck.write_checkpoint(m, str(tmp_path), train_op_bytes=op, stamp=1700000000)
    best = ck.write_checkpoint(m, str(tmp_path), best=True, train_op_bytes=op)
    assert sorted(os.listdir(tmp_path)) == ["net_1700000000", "net_BEST", "net_LAST", "net_train_op_BEST",
                                            "net_train_op_LAST"]            # deepnet/util.py:23-53
    assert os.path.basename(last) == "net_LAST" and os.path.basename(best) == "net_BEST"
    with gzip.open(os.path.join(tmp_path, "net_train_op_LAST"), "rb") as fh:
        stored = fh.read()
    assert ck.operation_current_step(stored) == 1234
    parsed = M["Operation"]()
    parsed.ParseFromString(stored)
    assert parsed.current_step == 1234 and parsed.batchsize == 100 and parsed.optimizer == 4
    np.testing.assert_array_equal(ck.read_model(last).get_edge_param("v", "h"),
                                  np.arange(6, dtype=np.float32).reshape(3, 2))


@pytest.mark.gpu
def test_trained_rbm_survives_a_checkpoint(cm, tmp_path):
    from deepnet_b200 import configs
    from deepnet_b200.fused_rbm import FusedRBM
    cfg = configs.build(0, cases=400, dims_scale=0.25)
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    B = cfg["batchsize"]
    mk = lambda w: FusedRBM(cm, V, H, B, w, cfg["hyperparams"], edge_hyperparams=cfg["edges"][0].get("hyperparams"),
                            binary_data=True, seed=cfg["seed"])
    eng = mk(cfg["edges"][0]["weight"])
    data = cm.CUDAMatrix(cfg["data"])
    for step in range(3):
        eng.TrainOneBatch(step, data.slice(step * B, (step + 1) * B))
    path = ck.write_checkpoint(ck.model_from_rbm(eng, "rbm"), str(tmp_path))
    other = mk(np.zeros((V, H), np.float32))
    ck.load_into_rbm(other, ck.read_model(path))
    for a, b in ((eng.W, other.W), (eng.bv, other.bv), (eng.bh, other.bh)):
        np.testing.assert_array_equal(np.array(a.asarray()), np.array(b.asarray()))
    # the restored engine computes the same hidden representation
    np.testing.assert_array_equal(eng.Inference(data.slice(0, B)), other.Inference(data.slice(0, B)))
