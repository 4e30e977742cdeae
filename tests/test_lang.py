import json

import pytest

from pccl_b200.lang import (ALGORITHMS, Chunk, CollectiveIR, Device, DeviceType, DirectedGraph, Link,
                            LoweringError, PrimitiveOpType, build, check_lowered_deadlock_free, lower,
                            port_load, to_schedule, verify)


def test_graph_basics():
    g = DirectedGraph()
    for n in (10, 20, 30, 40):
        g.add_node(n)
    g.add_edge(10, 20); g.add_edge(20, 30); g.add_edge(10, 30)
    assert g.is_acyclic()
    order = g.topological_sort()
    assert order.index(10) < order.index(20) < order.index(30)
    assert sorted(map(sorted, g.get_connected_components())) == [[10, 20, 30], [40]]
    assert g.get_predecessors(30) == [20, 10] or sorted(g.get_predecessors(30)) == [10, 20]
    g.add_edge(30, 10)
    assert not g.is_acyclic()
    with pytest.raises(ValueError):
        g.topological_sort()
    assert g.remove_edge(30, 10) and g.is_acyclic()
    with pytest.raises(ValueError):
        g.add_edge(10, 99)


def test_graph_ids_are_the_callers():
    # device ids need not be 0..n-1 in insertion order
    ir = CollectiveIR("t")
    for d in (7, 3):
        ir.add_device(Device(d, DeviceType.CUDA))
    ir.add_link(Link(7, 3))
    assert ir.validate_topology()
    assert ir.get_device_bandwidth_matrix()[(3, 7)] == ir.get_device_bandwidth_matrix()[(7, 3)]


def test_ir_builder_and_reference_api():
    ir = CollectiveIR("two_rank_sum", "allreduce", units=1, buffers={"input": 1, "output": 1, "scratch": 1})
    ir.add_device(Device(0, DeviceType.CPU, 1e11, 0)); ir.add_device(Device(1, DeviceType.CPU, 1e11, 0))
    ir.add_link(Link(0, 1, 1e10, 1e-5))
    ir.set_precondition([Chunk({0}, 0, 1, 0), Chunk({1}, 1, 1, 0)])
    a = ir.create_operation(PrimitiveOpType.COPY, Chunk({0}, 0, 1, 0, "input"), Chunk({0}, 0, 1, 0, "output"))
    b = ir.create_operation(PrimitiveOpType.COPY, Chunk({1}, 1, 1, 0, "input"), Chunk({1}, 0, 1, 0, "scratch"))
    c = ir.create_operation(PrimitiveOpType.REDUCE, Chunk({1}, 0, 1, 0, "scratch"), Chunk({0, 1}, 0, 1, 0, "output"),
                            dependencies=[a, b])
    ir.set_postcondition([Chunk({0, 1}, 0, 1, 0, "output")])
    assert ir.validate_dag() and ir.validate_topology()
    assert [o.op_id for o in ir.get_operation_sequence()][-1] == c
    assert verify(ir, check_relaunch=False).ok        # rank 1 only sends: fine for one launch
    assert any("relaunch" in e for e in verify(ir).errors)
    with pytest.raises(ValueError):
        ir.create_operation(PrimitiveOpType.COPY, dependencies=[999])


@pytest.mark.parametrize("name", sorted(ALGORITHMS))
@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_every_algorithm_verifies_and_lowers(name, n):
    if (name in ("recursive_doubling_allgather", "halving_doubling_allreduce") and n & (n - 1)) or \
            (name in ("hierarchical_allreduce", "hierarchical_allgather") and n % 2):
        with pytest.raises(ValueError):
            build(name, n)
        return
    ir = build(name, n, channels=2)
    rep = verify(ir)
    assert rep.ok, rep.errors[:3]
    low = lower(ir)
    assert low["num_ranks"] == n and len(low["slot_counts"]) == low["num_slots"]
    assert check_lowered_deadlock_free(low)
    again = CollectiveIR.from_json(ir.to_json())
    assert verify(again).ok and lower(again) == low


@pytest.mark.parametrize("name", ["direct_allreduce", "direct_reduce_scatter", "direct_allgather"])
@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_pull_forms_use_no_scratch_and_stand_between_two_barriers(name, n):
    """``direct=True``: peers' inputs are read and peers' outputs written in place.  No scratch at all, every stream begins
    and ends with a barrier (inputs complete / every remote access over), the program verifies and lowers deadlock-free."""
    ir = build(name, n, channels=2, direct=True)
    assert ir.buffers["scratch"] == 0 and ir.name.endswith(("_pull", "_sym"))
    assert verify(ir).ok
    low = lower(ir)
    assert check_lowered_deadlock_free(low)
    ops = list(ir.ops.values())
    barriers = [op for op in ops if op.op_type == PrimitiveOpType.BARRIER]
    assert len(barriers) == 2 * 2 * n                  # entry and exit, per channel, per rank
    assert not any(getattr(c, "buffer", "") == "scratch" for op in ops for c in (op.src_chunk, op.tgt_chunk) if c is not None)


def test_verifier_catches_double_count_missing_data_and_races():
    ir = build("direct_reduce_scatter", 2)
    # reduce the same contribution twice
    red = [o for o in ir.ops.values() if o.op_type == PrimitiveOpType.REDUCE][0]
    ir.create_operation(PrimitiveOpType.REDUCE, red.src_chunk.copy(), red.tgt_chunk.copy(), dependencies=[red.op_id])
    rep = verify(ir, check_annotations=False)
    assert not rep.ok and any("twice" in e for e in rep.errors)

    ir = build("direct_allgather", 3)
    # drop one op's effect by pointing the postcondition at data nobody wrote
    ir.postcondition.append(Chunk({0}, 1, 1, 0, "scratch", origin=0))
    ir.buffers["scratch"] = 3
    bad = build("ring_allreduce", 3)
    victim = [o for o in bad.ops.values() if o.op_type == PrimitiveOpType.REDUCE][0]
    victim.dependencies.clear()
    for p in bad.op_dag.get_predecessors(victim.op_id):
        bad.op_dag.remove_edge(p, victim.op_id)
    rep = verify(bad)
    assert not rep.ok   # either reads undefined data or races with the producer


def test_port_load_of_direct_forms_is_balanced():
    n = 8
    for name in ("direct_reduce_scatter", "direct_allgather", "alltoall"):
        load = port_load(build(name, n))
        assert len({v for v in load.values()}) == 1
        assert load[0][0] == n - 1 and load[0][1] == n - 1
    ring = port_load(build("ring_allreduce", n))
    assert ring[0] == (2 * (n - 1), 2 * (n - 1))


def test_schedule_document_shape():
    doc = to_schedule(build("ring_allreduce", 2))
    text = json.dumps(doc)
    back = json.loads(text)
    assert back["lowered"]["num_ranks"] == 2 and back["attrs"]["block_units"] == back["units"]
    ins = back["lowered"]["programs"][0][0][0]
    assert len(ins) == 10


def test_lowering_rejects_missing_barrier_partner():
    ir = build("nvls_allreduce", 2)
    # remove rank 1's final barrier: rank 0's barrier then has no partner
    last = max(i for i, o in ir.ops.items() if o.op_type == PrimitiveOpType.BARRIER and o.executor == 1)
    del ir.ops[last]
    ir2 = CollectiveIR("broken", "allreduce", ir.units, buffers=ir.buffers, in_place=True)
    for d in ir.devices.values():
        ir2.add_device(d)
    remap = {}
    for i, o in ir.ops.items():
        remap[i] = ir2.create_operation(o.op_type, o.src_chunk, o.tgt_chunk, o.src_device, o.tgt_device,
                                        [remap[d] for d in o.dependencies if d in remap], o.metadata)
    with pytest.raises(LoweringError):
        lower(ir2)


def test_reference_module_names_resolve_and_cluster_operator_helpers_work(tmp_path):
    import pccl.lang.chunk as chunk
    import pccl.lang.cluster as cluster
    import pccl.lang.operator as operator
    import pccl.lang.topology as topology
    from pccl.lang.utils.graph import DirectedGraph as DG
    from pccl_b200.lang import Cluster, Operator, DirectedGraph, build, verify
    assert DG is DirectedGraph and chunk.CollectiveIR is not None and topology.Topology is not None
    assert cluster.Cluster is Cluster and operator.Operator is Operator
    # a ring cluster stamped onto a ring program verifies; the same program on too small a cluster is refused
    ir = Cluster.ring(4).apply(build("ring_allreduce", 4, channels=2))
    verify(ir).raise_if_failed()
    assert len(ir.links) == 8 and ir.attrs["cluster"] == "ring4"
    with pytest.raises(ValueError):
        Cluster.ring(2).apply(build("ring_allreduce", 4))
    # cluster <-> synthesiser topology
    topo = Cluster.nvswitch(8).to_topology()
    assert topo.n == 8 and len(topo.link_bw) == 56
    assert Cluster.from_topology(topology.Topology.ring(4)).world_size == 4
    # operators: from the library, synthesised, saved as a schedule file
    op = Operator.from_algorithm("direct_allreduce", 4)
    doc = op.schedule()
    assert doc["collective"] == "allreduce" and op.schedule() is doc
    import json
    assert json.load(open(op.save(str(tmp_path / "op.json"))))["world_size"] == 4
    syn = Operator.synthesized("allgather", Cluster.ring(4).to_topology(), 1 << 20)
    assert syn.collective == "allgather" and syn.ir.attrs["synthesized"]
    with pytest.raises(RuntimeError):
        op(None)                      # not registered with an engine


def test_default_channel_count_comes_from_the_environment(monkeypatch):
    from pccl_b200.lang import build, to_schedule

    def streams(doc):
        return doc["lowered"]["num_channels"]
    monkeypatch.delenv("PCCL_CHANNELS", raising=False)
    one = streams(to_schedule(build("ring_allreduce", 4)))
    monkeypatch.setenv("PCCL_CHANNELS", "3")
    assert streams(to_schedule(build("ring_allreduce", 4))) == 3 * one
    assert streams(to_schedule(build("ring_allreduce", 4, channels=1))) == one      # an explicit argument wins


def test_operator_best_picks_by_the_cost_model():
    from pccl_b200.lang import Operator
    from pccl_b200.synth import Topology
    assert Operator.best("allreduce", Topology.nvswitch(8), 1 << 10).name == "oneshot_allreduce"
    assert Operator.best("allreduce", Topology.nvswitch(8), 64 << 20).name == "direct_allreduce"
    with pytest.raises(ValueError):
        Operator.best("alltoall", Topology.ring(4), 1 << 20)
    op = Operator.best("alltoall", Topology.ring(4), 1 << 20, include_milp=True)
    assert op.name.startswith("milp_alltoall") and op.estimate.steps >= 2 and op.schedule()["collective"] == "alltoall"


def test_verifier_rejects_a_sender_that_nothing_holds_back():
    """Run again and again, a rank that only sends gets ahead of its receiver and overwrites workspace that is still
    being read; the verifier wants a tie from the receiver back to the sender."""
    from pccl_b200.lang import relaunch_hazards

    def program(ack: bool) -> CollectiveIR:
        ir = CollectiveIR("one_way", "send_recv", units=1, buffers={"input": 1, "output": 1, "scratch": 1})
        ir.add_device(Device(0, DeviceType.CPU)); ir.add_device(Device(1, DeviceType.CPU))
        ir.add_link(Link(0, 1))
        ir.set_precondition([Chunk({0}, 0, 1, 0, "input")])
        ir.set_postcondition([Chunk({0}, 1, 1, 0, "output")])
        push = ir.copy(Chunk({0}, 0, 1, 0, "input"), Chunk({0}, 1, 1, 0, "scratch"))
        took = ir.copy(Chunk({0}, 1, 1, 0, "scratch"), Chunk({0}, 1, 1, 0, "output"), deps=[push])
        if ack:
            ir.get_notified(1, 0, deps=[ir.notify(1, 0, deps=[took])])
        return ir
    bare = program(False)
    assert relaunch_hazards(bare) == [(0, 1)]
    rep = verify(bare)
    assert not rep.ok and "relaunch" in rep.errors[0]
    assert verify(bare, check_relaunch=False).ok          # a program that is launched once may leave it out
    assert verify(program(True)).ok and relaunch_hazards(program(True)) == []
    # the library's one-way programs carry the acknowledgement
    for name in ("send_recv", "broadcast", "reduce", "scatter", "gather"):
        assert relaunch_hazards(build(name, 4)) == []


def test_every_module_is_reachable_under_the_reference_package_name():
    import importlib
    import pccl
    import pccl_b200.synth
    assert importlib.import_module("pccl.synth") is pccl_b200.synth and pccl_b200.synth.__spec__.name == "pccl_b200.synth"
    assert importlib.import_module("pccl.engine.elastic").join_as_spare is not None
    assert importlib.import_module("pccl.synth.local_node").LocalNode is pccl_b200.synth.LocalNode
    assert importlib.import_module("pccl.lang.chunk").CollectiveIR is pccl.lang.CollectiveIR      # the package's own files win
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("pccl.no_such_module")


def test_regop_checks_schedule_documents_too(tmp_path):
    import json as _json
    from pccl_b200.engine import Engine
    from pccl_b200.lang import VerificationError, add_acknowledgements, to_schedule
    ir = CollectiveIR("one_way", "send_recv", units=1, buffers={"input": 1, "output": 1, "scratch": 1})
    ir.add_device(Device(0, DeviceType.CPU)); ir.add_device(Device(1, DeviceType.CPU)); ir.add_link(Link(0, 1))
    ir.set_precondition([Chunk({0}, 0, 1, 0, "input")]); ir.set_postcondition([Chunk({0}, 1, 1, 0, "output")])
    push = ir.copy(Chunk({0}, 0, 1, 0, "input"), Chunk({0}, 1, 1, 0, "scratch"))
    ir.copy(Chunk({0}, 1, 1, 0, "scratch"), Chunk({0}, 1, 1, 0, "output"), deps=[push])
    doc = to_schedule(ir)
    path = tmp_path / "one_way.json"
    path.write_text(_json.dumps(doc))
    e = Engine(0, 2); e.initEngine("cpu")
    for form in (doc, _json.dumps(doc), str(path)):
        with pytest.raises(VerificationError, match="relaunch"):
            e.regOp("bad", form)
    e.regOp("as_it_is", doc, check=False)
    assert add_acknowledgements(ir) == 1
    e.regOp("good", to_schedule(ir))
