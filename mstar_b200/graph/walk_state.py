"""Run-time state of one request's walk on one worker: which inputs every node holds, which nodes are ready,
where loops stand, and what to route when a node completes.

One ``WalkState`` replaces the reference's per-request deep copy of the graph with its nested state registries
(``GraphStateRegistry`` / ``LoopStateRegistry``, mstar/graph/base.py:644-787) and ``WorkerGraphIO``
(mstar/graph/graph_io.py:10-214); the declarative graph stays shared and immutable.

Semantics kept from the reference:
  * a node is ready when every declared input has arrived (streaming inputs may still be missing:
    ``ready_for_streaming``);
  * a second arrival of an input that the current iteration already holds is buffered for the next iteration;
  * a loop iteration ends when every entity of its body has completed; then either the loop ends (iteration
    budget used up, or ``stop_loop`` was called) — its ``outputs`` leave with the last iteration's tensors, its
    ``accumulated_outputs`` with all iterations' tensors, loop-back signals are dropped — or the next iteration
    starts: buffered inputs become current and the inputs that came from outside the loop are delivered again;
  * speculation: while iteration N of a self-feeding loop node still runs, the worker may ask whether iteration
    N+1 could start as soon as N's own outputs exist (``can_speculate``), mark it (``begin_speculation``) and
    undo the mark when a stop arrives (``rollback_speculation``).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .ir import GraphEdge, GraphNode, GraphSection, Loop, SPECIAL_DESTINATIONS, entities_of


@dataclass
class Completion:
    route: list[GraphEdge] = field(default_factory=list)       # edges for other workers / the client / nowhere
    delivered: list[GraphEdge] = field(default_factory=list)   # edges consumed by nodes of this walk state
    dropped: list[GraphEdge] = field(default_factory=list)     # loop-back edges of a loop that just ended
    finished_loops: list[str] = field(default_factory=list)
    advanced_loops: list[str] = field(default_factory=list)
    walk_done: bool = False


class _NodeState:
    __slots__ = ("decl", "cur", "nxt", "done", "running", "speculating", "scope")

    def __init__(self, decl: GraphNode, scope: "_Scope"):
        self.decl, self.scope = decl, scope
        self.cur: dict[str, GraphEdge] = {}
        self.nxt: dict[str, GraphEdge] = {}
        self.done = False          # completed in the current iteration
        self.running = False       # handed to an engine, not completed yet
        self.speculating = False   # iteration N+1 was launched before N completed

    def missing(self) -> set[str]:
        return self.decl.input_names - set(self.cur)

    def is_ready(self) -> bool:
        return not self.missing()

    def is_ready_for_streaming(self) -> bool:
        return self.missing() <= self.decl.streaming_inputs


class _Scope:
    """Top level of a walk, or the body of one loop."""

    def __init__(self, section: GraphSection, parent: "_Scope | None", loop: Loop | None):
        self.parent, self.loop = parent, loop
        self.entity_names = [e.name for e in entities_of(section)]
        self.completed: set[str] = set()
        # loop bookkeeping
        self.curr_iter = 0
        self.finish = False
        self.done = False
        self.saved_inputs: dict[tuple[str, str], GraphEdge] = {}
        self.last_outputs: dict[str, list] = {}
        self.accumulated: dict[str, list] = {}

    def all_complete(self) -> bool:
        return len(self.completed) == len(self.entity_names)


class WalkState:
    def __init__(self, section: GraphSection, request_id: str = "", on_release=None):
        """``on_release(edge)`` is called when a consumed input edge is dropped (tensor refcount hook)."""
        self.section, self.request_id, self.on_release = section, request_id, on_release
        self.nodes: dict[str, _NodeState] = {}
        self.scopes: dict[str, _Scope] = {}          # loop name -> scope
        self.top = _Scope(section, None, None)
        self._build(section, self.top)
        self.done = False

    def _build(self, section: GraphSection, scope: _Scope) -> None:
        for ent in entities_of(section):
            if isinstance(ent, GraphNode):
                self.nodes[ent.name] = _NodeState(ent, scope)
            else:
                inner = _Scope(ent.section, scope, ent)
                self.scopes[ent.name] = inner
                self._build(ent.section, inner)

    # ------------------------------------------------------------------ queries
    def has_node(self, name: str) -> bool:
        return name in self.nodes

    def ready_nodes(self, allow_streaming: bool = True) -> list[str]:
        out = []
        for name, st in self.nodes.items():
            if st.done or st.running or st.scope.done:
                continue
            if st.is_ready() or (allow_streaming and st.decl.consumes_stream and st.is_ready_for_streaming()
                                 and st.missing()):
                out.append(name)
        return out

    def inputs_of(self, name: str) -> dict[str, GraphEdge]:
        return dict(self.nodes[name].cur)

    def loop_indices(self) -> dict[str, int]:
        return {n: s.curr_iter for n, s in self.scopes.items()}

    def enclosing_loops(self, node: str) -> list[str]:
        out, sc = [], self.nodes[node].scope
        while sc is not None and sc.loop is not None:
            out.append(sc.loop.name)
            sc = sc.parent
        return out

    # ------------------------------------------------------------------ ingest
    def ingest(self, edge: GraphEdge, can_buffer: bool = True) -> bool:
        """Deliver an edge to its consumer node. False when this walk state has no use for it (unknown node or
        input name, or the slot is already full and buffering is not allowed)."""
        st = self.nodes.get(edge.next_node)
        if st is None or edge.name not in st.decl.input_names:
            return False
        if edge.name not in st.cur:
            st.cur[edge.name] = edge
        elif can_buffer and edge.name not in st.nxt:
            st.nxt[edge.name] = edge
        else:
            return False
        # remember inputs that cross into a loop from outside: they are delivered again every iteration
        sc = st.scope
        # (stream chunks are consumed once: each iteration gets a fresh chunk from the stream buffer)
        streaming = edge.is_streaming or edge.name in st.decl.streaming_inputs
        while sc is not None and sc.loop is not None and not streaming:
            if edge.key() in sc.loop.external_inputs and edge.key() not in sc.saved_inputs:
                sc.saved_inputs[edge.key()] = edge
            sc = sc.parent
        return True

    def remove_input(self, node: str, name: str) -> GraphEdge | None:
        """Take an input back out of a node's current slot (a streaming chunk that goes back to its buffer)."""
        return self.nodes[node].cur.pop(name, None)

    def mark_running(self, node: str) -> None:
        self.nodes[node].running = True

    # ------------------------------------------------------------------ completion
    def stop_loop(self, loop_name: str) -> None:
        sc = self.scopes.get(loop_name)
        if sc is not None:
            sc.finish = True

    def complete(self, node: str, outputs: list[GraphEdge] | None = None, iterations: int = 1) -> Completion:
        """Node finished its forward for this iteration; ``outputs`` are its declared output edges with
        tensor_info filled in (defaults to the declaration's edges). ``iterations`` > 1: the execution covered
        that many iterations of the node's loop at once (a decode burst); the loop counter moves accordingly."""
        st = self.nodes[node]
        if iterations > 1 and st.scope.loop is not None:
            st.scope.curr_iter += iterations - 1
        res = Completion()
        outputs = list(st.decl.outputs) if outputs is None else list(outputs)
        st.running = False
        st.done = True
        st.speculating = False
        scope = st.scope
        scope.completed.add(node)
        self._cache_loop_outputs(scope, outputs)
        pending = outputs
        # walk outwards while scopes finish
        while True:
            if scope.loop is None:
                self._deliver(pending, res)
                if scope.all_complete():
                    self.done = True
                    res.walk_done = True
                return res
            if not scope.all_complete():
                self._deliver(pending, res)
                return res
            loop = scope.loop
            last = (scope.curr_iter + 1 >= loop.max_iters) or scope.finish
            if not last:
                self._deliver(pending, res)
                self._advance(scope)
                res.advanced_loops.append(loop.name)
                return res
            # the loop ends: loop-back signals die here, the loop's own outputs leave
            keep = []
            for e in pending:
                (res.dropped if e.key() in loop.loop_back_inputs else keep).append(e)
            self._deliver(keep, res)
            loop_out = []
            for decl in loop.outputs:
                e = decl.clone(with_tensors=False)
                e.tensor_info = list(scope.last_outputs.get(decl.name, []))
                loop_out.append(e)
            for decl in loop.accumulated_outputs:
                e = decl.clone(with_tensors=False)
                e.tensor_info = list(scope.accumulated.get(decl.name, []))
                loop_out.append(e)
            scope.done = True
            scope.last_outputs, scope.accumulated = {}, {}
            res.finished_loops.append(loop.name)
            parent = scope.parent
            parent.completed.add(loop.name)
            self._cache_loop_outputs(parent, loop_out)
            pending, scope = loop_out, parent

    def _cache_loop_outputs(self, scope: _Scope, edges: list[GraphEdge]) -> None:
        if scope.loop is None:
            return
        last_names = {e.name for e in scope.loop.outputs}
        acc_names = {e.name for e in scope.loop.accumulated_outputs}
        seen: set[str] = set()
        for e in edges:
            if e.name in seen:
                continue
            seen.add(e.name)
            if e.name in last_names:
                scope.last_outputs[e.name] = list(e.tensor_info)
            elif e.name in acc_names:
                scope.accumulated.setdefault(e.name, []).extend(e.tensor_info)

    def _deliver(self, edges: list[GraphEdge], res: Completion) -> None:
        for e in edges:
            if e.next_node in SPECIAL_DESTINATIONS or e.next_node not in self.nodes:
                res.route.append(e)
            elif self.ingest(e):
                res.delivered.append(e)
            else:
                res.route.append(e)

    def _advance(self, scope: _Scope) -> None:
        """Start the next iteration of ``scope``'s loop."""
        scope.curr_iter += 1
        scope.completed.clear()
        scope.last_outputs = {}
        self._reset_scope_nodes(scope, rotate=True)
        for e in list(scope.saved_inputs.values()):
            self.ingest(e.clone(), can_buffer=False)

    def _reset_scope_nodes(self, scope: _Scope, rotate: bool) -> None:
        for st in self.nodes.values():
            if st.scope is scope:
                if self.on_release is not None:
                    for e in st.cur.values():
                        if e.key() not in scope.saved_inputs:
                            self.on_release(e)
                st.cur = st.nxt if rotate else {}
                st.nxt = {}
                st.done = st.running = False
        for name, inner in self.scopes.items():
            if inner.parent is scope:
                # a nested loop starts over inside the new outer iteration
                inner.curr_iter, inner.finish, inner.done = 0, False, False
                inner.completed.clear()
                inner.saved_inputs.clear()
                inner.last_outputs, inner.accumulated = {}, {}
                self._reset_scope_nodes(inner, rotate=rotate)

    # ------------------------------------------------------------------ speculation
    def can_speculate(self, node: str, ahead: int = 1, chained: bool = False) -> bool:
        """May a further iteration of ``node`` be launched while earlier ones still run? True when the node sits
        alone in a loop that will go on, and every input of the new iteration is either its own loop-back output,
        an input from outside the loop (delivered again each iteration) or already buffered. ``ahead`` = iterations
        already launched and not completed (1: only the running one); ``chained`` allows a speculative launch on
        top of another speculative launch."""
        st = self.nodes[node]
        sc = st.scope
        if sc.loop is None or not st.decl.enable_async_scheduling or (st.speculating and not chained):
            return False
        if sc.finish or sc.curr_iter + ahead + 1 > sc.loop.max_iters:
            return False
        if len(sc.entity_names) != 1:
            return False
        own = {e.name for e in st.decl.outputs if e.next_node == node}
        saved = {k[0] for k in sc.saved_inputs if k[1] == node}
        need = st.decl.input_names - st.decl.streaming_inputs
        return need <= (own | saved | set(st.nxt))

    def begin_speculation(self, node: str) -> None:
        self.nodes[node].speculating = True

    def rollback_speculation(self, node: str) -> None:
        self.nodes[node].speculating = False

    def clear(self) -> None:
        for st in self.nodes.values():
            if self.on_release is not None:
                for e in list(st.cur.values()) + list(st.nxt.values()):
                    self.on_release(e)
            st.cur, st.nxt = {}, {}
            st.done = st.running = st.speculating = False
