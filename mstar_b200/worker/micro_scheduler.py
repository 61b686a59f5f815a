"""Picks the next (node, walk, requests) batch of a worker. Round-robin over (node, walk) pairs by default, or
strict priority order; respects per-node batch limits; requests that just failed an allocation are held for a
back-off period; tensor-parallel followers do not schedule at all but replay the leader's decisions in order.

Reference counterpart: ``MicroScheduler`` (mstar/worker/micro_scheduler.py:46-403: hold/backoff :129-134,
_try_schedule_tp_follow :140-209, get_next_batch :212-340, has_ready_excluding :342-392).
"""
from __future__ import annotations

import time
from collections import OrderedDict, deque

HOLD_SECONDS = 0.05


class MicroScheduler:
    def __init__(self, max_batch_size: int = 64, policy: str = "round_robin", priorities: dict | None = None,
                 is_tp_follower: bool = False):
        self.max_batch_size = max_batch_size
        self.policy = policy
        self.priorities = priorities or {}
        self.is_tp_follower = is_tp_follower
        # nodes whose batches replay the instance leader's decisions (None: every node); a follower rank's other
        # nodes (a codec or encoder placed on that rank alone) are scheduled here like on any worker
        self.follow_nodes: set | None = None
        self.ready: "OrderedDict[tuple[str, str], OrderedDict[str, None]]" = OrderedDict()
        self._rr: deque = deque()
        self._held: dict[str, float] = {}
        self._tp_queue: deque = deque()          # leader decisions waiting to be replayed
        self._follow_wait = None                  # (decision, since, warned): a decision that cannot be replayed yet
        self.stalled = None
        self.node_limits: dict[str, int] = {}
        self.limit_fn = None                      # optional (node, walk) -> largest batch the node accepts
        # optional (node, walk, ready request ids, seconds since the first of them became ready) -> True to hold the
        # batch back a little longer so that requests about to become ready join it
        self.defer_fn = None
        self._first_ready: dict[tuple[str, str], float] = {}

    # ---- bookkeeping ----
    def mark_ready(self, node: str, walk: str, request_id: str) -> None:
        key = (node, walk)
        if key not in self.ready:
            self.ready[key] = OrderedDict()
            self._rr.append(key)
        if not self.ready[key]:
            self._first_ready[key] = time.monotonic()
        self.ready[key][request_id] = None

    def unmark(self, node: str, walk: str, request_id: str) -> None:
        q = self.ready.get((node, walk))
        if q is not None:
            q.pop(request_id, None)

    def remove_request(self, request_id: str) -> None:
        for q in self.ready.values():
            q.pop(request_id, None)
        self._held.pop(request_id, None)

    def hold(self, request_ids, seconds: float = HOLD_SECONDS) -> None:
        until = time.monotonic() + seconds
        for r in request_ids:
            self._held[r] = until

    def push_tp_decision(self, node: str, walk: str, request_ids: list[str]) -> None:
        self._tp_queue.append((node, walk, list(request_ids)))

    def _eligible(self, key) -> list[str]:
        now = time.monotonic()
        out = []
        for r in self.ready.get(key, ()):
            t = self._held.get(r)
            if t is not None:
                if t > now:
                    continue
                del self._held[r]
            out.append(r)
        return out

    # ---- decisions ----
    def get_next_batch(self, exclude: set | None = None):
        """(node, walk, request_ids) or None."""
        if self.is_tp_follower:
            nxt = self._follow()
            if nxt is not None or self.follow_nodes is None:
                return nxt
        keys = [k for k in self._rr if self.ready.get(k)]
        if self.is_tp_follower:
            keys = [k for k in keys if k[0] not in self.follow_nodes]
        if not keys:
            return None
        if self.policy == "priority":
            keys.sort(key=lambda k: -self.priorities.get(k[0], 0))
        for key in keys:
            if exclude and key in exclude:
                continue
            rids = self._eligible(key)
            if not rids:
                continue
            if self.defer_fn is not None and len(rids) < self.max_batch_size and self.defer_fn(
                    key[0], key[1], rids, time.monotonic() - self._first_ready.get(key, 0.0)):
                continue
            limit = min(self.max_batch_size, self.node_limits.get(key[0], self.max_batch_size))
            if self.limit_fn is not None:
                limit = max(1, min(limit, int(self.limit_fn(key[0], key[1]))))
            rids = rids[:limit]
            for r in rids:
                self.ready[key].pop(r, None)
            if self.ready[key]:
                self._first_ready[key] = time.monotonic()
            if self.policy == "round_robin":
                self._rr.remove(key)
                self._rr.append(key)
            return key[0], key[1], rids
        return None

    def _follow(self):
        """Replay the leader's next decision once every request in it is ready here too."""
        if not self._tp_queue:
            return None
        node, walk, rids = self._tp_queue[0]
        q = self.ready.get((node, walk), {})
        if not all(r in q for r in rids):
            now = time.monotonic()
            if self._follow_wait is None or self._follow_wait[0] is not self._tp_queue[0]:
                self._follow_wait = (self._tp_queue[0], now, False)
            elif now - self._follow_wait[1] > 5.0 and not self._follow_wait[2]:
                self._follow_wait = (self._tp_queue[0], self._follow_wait[1], True)
                self.stalled = (node, walk, list(rids))          # the worker adds what the requests still miss
                import logging
                logging.getLogger("mstar.worker").warning(
                    "lockstep: the leader's batch %s:%s %s waits for requests that are not ready on this rank: %s "
                    "(ready here: %s)", node, walk, rids, [r for r in rids if r not in q],
                    {k: list(v) for k, v in self.ready.items() if v})
            return None
        self._tp_queue.popleft()
        for r in rids:
            q.pop(r, None)
        return node, walk, rids

    def has_ready_excluding(self, key) -> bool:
        return any(k != key and self._eligible(k) for k in self.ready)

    def has_ready(self) -> bool:
        return any(self._eligible(k) for k in self.ready)
