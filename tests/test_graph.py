"""Graph IR and walk-state semantics: sequential / parallel composition, loops (iteration budget, stop signal,
last-iteration vs accumulated outputs, re-delivery of outside inputs), nested loops, streaming readiness,
speculation gate."""
from mstar_b200.graph import (EMIT_TO_CLIENT, GraphEdge, GraphNode, Loop, Parallel, Sequential, TensorPointerInfo,
                              WalkState)


def _t(tag):
    return TensorPointerInfo(dims=[1], dtype="int64", nbytes=8, uuid=tag)


def _with(edges, tag):
    out = []
    for e in edges:
        c = e.clone(with_tensors=False)
        c.tensor_info = [_t(f"{e.name}:{tag}")]
        out.append(c)
    return out


def test_sequential_signature_and_flow():
    a = GraphNode("a", {"x"}, [GraphEdge("b", "h")])
    b = GraphNode("b", {"h"}, [GraphEdge(EMIT_TO_CLIENT, "y", output_modality="text")])
    sec = Sequential([a, b])
    sig = sec.signature()
    assert sig.ext_inputs == {("x", "a")} and [e.name for e in sig.ext_outputs] == ["y"] and not sig.loop_back
    ws = WalkState(sec)
    assert ws.ready_nodes() == []
    assert ws.ingest(GraphEdge("a", "x"))
    assert not ws.ingest(GraphEdge("a", "nope")) and not ws.ingest(GraphEdge("zzz", "x"))
    assert ws.ready_nodes() == ["a"]
    c = ws.complete("a", _with(a.outputs, 0))
    assert [e.name for e in c.delivered] == ["h"] and not c.route and not c.walk_done
    assert ws.ready_nodes() == ["b"]
    c = ws.complete("b", _with(b.outputs, 0))
    assert [e.next_node for e in c.route] == [EMIT_TO_CLIENT] and c.walk_done and ws.done


def test_parallel_join():
    enc1 = GraphNode("enc1", {"img"}, [GraphEdge("llm", "e1")])
    enc2 = GraphNode("enc2", {"aud"}, [GraphEdge("llm", "e2")])
    llm = GraphNode("llm", {"e1", "e2"}, [GraphEdge(EMIT_TO_CLIENT, "out")])
    sec = Sequential([Parallel([enc1, enc2]), llm])
    assert sec.signature().ext_inputs == {("img", "enc1"), ("aud", "enc2")}
    ws = WalkState(sec)
    ws.ingest(GraphEdge("enc1", "img"))
    ws.ingest(GraphEdge("enc2", "aud"))
    assert sorted(ws.ready_nodes()) == ["enc1", "enc2"]
    ws.complete("enc1", _with(enc1.outputs, 0))
    assert "llm" not in ws.ready_nodes()
    ws.complete("enc2", _with(enc2.outputs, 0))
    assert ws.ready_nodes() == ["llm"]


def _decode_loop(max_iters=4):
    llm = GraphNode("LLM", {"tok", "ctx"},
                    [GraphEdge("LLM", "tok"), GraphEdge(EMIT_TO_CLIENT, "new_token", conductor_new_token=True)])
    loop = Loop(llm, max_iters=max_iters, name="decode_loop",
                outputs=[GraphEdge("post", "tok")], accumulated_outputs=[GraphEdge("post", "new_token")])
    post = GraphNode("post", {"tok", "new_token"}, [GraphEdge(EMIT_TO_CLIENT, "final")])
    return llm, loop, post, Sequential([loop, post])


def test_loop_runs_max_iters_and_emits_last_and_accumulated():
    llm, loop, post, sec = _decode_loop(3)
    assert loop.loop_back_inputs == {("tok", "LLM")} and loop.external_inputs == {("ctx", "LLM")}
    ws = WalkState(sec)
    ws.ingest(GraphEdge("LLM", "tok", [_t("tok:init")]))
    ws.ingest(GraphEdge("LLM", "ctx", [_t("ctx")]))
    for it in range(3):
        assert ws.ready_nodes() == ["LLM"], it
        assert ws.loop_indices() == {"decode_loop": it}
        assert ws.inputs_of("LLM")["ctx"].tensor_info[0].uuid == "ctx"      # outside input is delivered every iter
        ws.mark_running("LLM")
        assert ws.ready_nodes() == []
        c = ws.complete("LLM", _with(llm.outputs, it))
        assert [e.name for e in c.route if e.next_node == EMIT_TO_CLIENT] == ["new_token"]
        if it < 2:
            assert c.advanced_loops == ["decode_loop"] and not c.finished_loops
            assert ws.inputs_of("LLM")["tok"].tensor_info[0].uuid == f"tok:{it}"
        else:
            assert c.finished_loops == ["decode_loop"] and [e.name for e in c.dropped] == ["tok"]
    assert ws.ready_nodes() == ["post"]
    ins = ws.inputs_of("post")
    assert [t.uuid for t in ins["tok"].tensor_info] == ["tok:2"]
    assert [t.uuid for t in ins["new_token"].tensor_info] == ["new_token:0", "new_token:1", "new_token:2"]


def test_stop_loop_ends_after_current_iteration():
    llm, loop, post, sec = _decode_loop(100)
    ws = WalkState(sec)
    ws.ingest(GraphEdge("LLM", "tok"))
    ws.ingest(GraphEdge("LLM", "ctx"))
    ws.complete("LLM", _with(llm.outputs, 0))
    ws.stop_loop("decode_loop")
    c = ws.complete("LLM", _with(llm.outputs, 1))
    assert c.finished_loops == ["decode_loop"]
    assert ws.ready_nodes() == ["post"]
    assert len(ws.inputs_of("post")["new_token"].tensor_info) == 2


def test_nested_loops_restart_inner_each_outer_iteration():
    inner_node = GraphNode("step", {"z", "cond"}, [GraphEdge("step", "z")])
    inner = Loop(inner_node, max_iters=2, name="inner", outputs=[GraphEdge("outer_tail", "z")])
    tail = GraphNode("outer_tail", {"z"}, [GraphEdge("step", "z"), GraphEdge(EMIT_TO_CLIENT, "img")])
    outer = Loop(Sequential([inner, tail]), max_iters=2, name="outer", outputs=[GraphEdge(EMIT_TO_CLIENT, "img")])
    ws = WalkState(outer)
    ws.ingest(GraphEdge("step", "z", [_t("z0")]))
    ws.ingest(GraphEdge("step", "cond", [_t("cond")]))
    trace = []
    for _ in range(20):
        r = ws.ready_nodes()
        if not r:
            break
        n = r[0]
        trace.append((n, dict(ws.loop_indices())))
        c = ws.complete(n, _with(ws.nodes[n].decl.outputs, len(trace)))
        if c.walk_done:
            break
    assert [t[0] for t in trace] == ["step", "step", "outer_tail", "step", "step", "outer_tail"]
    assert trace[3][1] == {"inner": 0, "outer": 1}
    assert ws.done


def test_streaming_node_ready_without_stream_input():
    codec = GraphNode("codec", {"codes", "cfg"}, [GraphEdge(EMIT_TO_CLIENT, "audio")], streaming_inputs={"codes"})
    ws = WalkState(codec)
    ws.ingest(GraphEdge("codec", "cfg"))
    assert ws.ready_nodes() == ["codec"] and ws.ready_nodes(allow_streaming=False) == []
    ws.ingest(GraphEdge("codec", "codes", is_streaming=True))
    assert ws.ready_nodes(allow_streaming=False) == ["codec"]
    assert ws.remove_input("codec", "codes") is not None
    assert ws.ready_nodes(allow_streaming=False) == []


def test_speculation_gate():
    llm, loop, post, sec = _decode_loop(3)
    ws = WalkState(sec)
    ws.ingest(GraphEdge("LLM", "tok"))
    ws.ingest(GraphEdge("LLM", "ctx"))
    ws.mark_running("LLM")
    assert ws.can_speculate("LLM")
    ws.begin_speculation("LLM")
    assert not ws.can_speculate("LLM")            # one step deep
    ws.complete("LLM", _with(llm.outputs, 0))
    ws.mark_running("LLM")
    assert ws.can_speculate("LLM")
    ws.complete("LLM", _with(llm.outputs, 1))     # iteration index 2 is the last one
    assert not ws.can_speculate("LLM")
    ws2 = WalkState(sec)
    ws2.stop_loop("decode_loop")
    assert not ws2.can_speculate("LLM")
    assert not WalkState(sec).can_speculate("post")


def test_release_hook_called_for_consumed_inputs():
    released = []
    llm, loop, post, sec = _decode_loop(2)
    ws = WalkState(sec, on_release=lambda e: released.append(e.name))
    ws.ingest(GraphEdge("LLM", "tok"))
    ws.ingest(GraphEdge("LLM", "ctx"))
    ws.complete("LLM", _with(llm.outputs, 0))
    assert released == ["tok"]                     # ctx is kept for the next iteration
