"""Cluster manager, heartbeat-based failure detection and resource scheduling
(src/distributed/cluster.rs:30-719).

The heartbeat path is host-only: nodes report liveness (directly or through a key-value store such as
``torch.distributed.TCPStore``); a monitor thread marks nodes ``FAILED`` after ``node_timeout`` without a
beat and the manager's failover handler picks a replacement, moves the failed node's jobs and rebuilds
the affected process-group membership (the reference leaves the last two as no-ops, cluster.rs:332-405).
Nothing here touches a GPU: failures are detected and injected on the host.
"""
from __future__ import annotations

import enum
import json
import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional


class NodeStatus(enum.Enum):
    """Life-cycle state of a cluster node as seen by the heartbeat monitor."""

    ACTIVE = "active"
    IDLE = "idle"
    BUSY = "busy"
    FAILED = "failed"
    DRAINING = "draining"


class ClusterTopology(enum.Enum):
    """How the nodes of a cluster are connected (src/distributed/cluster.rs)."""

    FLAT = "flat"
    TREE = "tree"
    RING = "ring"
    CUSTOM = "custom"


class SchedulingPolicy(enum.Enum):
    """How the cluster manager picks nodes for a job."""

    FIRST_FIT = "first_fit"
    BEST_FIT = "best_fit"
    LOAD_BALANCING = "load_balancing"
    LOCALITY_AWARE = "locality_aware"


@dataclass
class NodeCapabilities:
    gpus: int = 8
    gpu_memory_gb: float = 180.0
    cpu_cores: int = 64
    memory_gb: float = 1024.0
    interconnect: str = "nvlink5"


@dataclass
class NodeInfo:
    node_id: int
    address: str = "127.0.0.1"
    port: int = 29500
    capabilities: NodeCapabilities = field(default_factory=NodeCapabilities)
    status: NodeStatus = NodeStatus.ACTIVE
    last_heartbeat: float = field(default_factory=time.monotonic)
    load: float = 0.0
    rack: str = "r0"
    jobs: List[str] = field(default_factory=list)


@dataclass
class FaultToleranceConfig:
    enable_failover: bool = True
    heartbeat_interval: float = 1.0
    node_timeout: float = 5.0
    max_retries: int = 3
    retry_delay: float = 0.1
    checkpoint_frequency: int = 1000


@dataclass
class ClusterConfig:
    name: str = "cluster"
    topology: ClusterTopology = ClusterTopology.FLAT
    fault_tolerance: FaultToleranceConfig = field(default_factory=FaultToleranceConfig)
    scheduling: SchedulingPolicy = SchedulingPolicy.LOAD_BALANCING

    def to_json(self) -> str:
        d = asdict(self)
        d["topology"], d["scheduling"] = self.topology.value, self.scheduling.value
        return json.dumps(d)

    @staticmethod
    def from_json(s: str) -> "ClusterConfig":
        d = json.loads(s)
        return ClusterConfig(d["name"], ClusterTopology(d["topology"]), FaultToleranceConfig(**d["fault_tolerance"]),
                             SchedulingPolicy(d["scheduling"]))


class HeartbeatMonitor:
    """Marks nodes failed when ``now - last_heartbeat > node_timeout`` and calls ``on_failure(node_id)`` once."""

    def __init__(self, nodes: Dict[int, NodeInfo], config: FaultToleranceConfig, on_failure: Callable[[int], None],
                 clock: Callable[[], float] = time.monotonic):
        self.nodes, self.config, self.on_failure, self.clock = nodes, config, on_failure, clock
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()

    def beat(self, node_id: int) -> None:
        with self._lock:
            n = self.nodes[node_id]
            n.last_heartbeat = self.clock()
            if n.status is NodeStatus.FAILED:
                n.status = NodeStatus.ACTIVE   # node came back

    def check_once(self) -> List[int]:
        failed = []
        now = self.clock()
        with self._lock:
            for n in self.nodes.values():
                if n.status is not NodeStatus.FAILED and now - n.last_heartbeat > self.config.node_timeout:
                    n.status = NodeStatus.FAILED
                    failed.append(n.node_id)
        for nid in failed:
            self.on_failure(nid)
        return failed

    def _run(self) -> None:
        while not self._stop.wait(self.config.heartbeat_interval):
            self.check_once()

    def start(self) -> None:
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
            self._thread = None


class StoreHeartbeat:
    """Liveness through a shared key-value store (``set/get`` of ``hb/<rank>`` = wall-clock seconds), for ranks
    of a ``torch.distributed`` job: each rank calls ``beat()`` between steps, any rank can ask ``dead_ranks()``."""

    def __init__(self, store, rank: int, world_size: int, timeout: float = 5.0, clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world_size, self.timeout, self.clock = store, rank, world_size, timeout, clock

    def beat(self) -> None:
        self.store.set(f"hb/{self.rank}", str(self.clock()))

    def dead_ranks(self) -> List[int]:
        now, dead = self.clock(), []
        for r in range(self.world_size):
            try:
                raw = self.store.get(f"hb/{r}")
                last = float(raw.decode() if hasattr(raw, "decode") else raw)
            except Exception:  # noqa: BLE001  (key never written)
                dead.append(r)
                continue
            if now - last > self.timeout:
                dead.append(r)
        return dead


class ResourceScheduler:
    def __init__(self, policy: SchedulingPolicy = SchedulingPolicy.LOAD_BALANCING):
        self.policy = policy

    def select(self, nodes: List[NodeInfo], gpus_needed: int = 1, prefer_rack: Optional[str] = None) -> Optional[NodeInfo]:
        ok = [n for n in nodes if n.status in (NodeStatus.ACTIVE, NodeStatus.IDLE) and n.capabilities.gpus >= gpus_needed]
        if not ok:
            return None
        if self.policy is SchedulingPolicy.FIRST_FIT:
            return ok[0]
        if self.policy is SchedulingPolicy.BEST_FIT:
            return min(ok, key=lambda n: (n.capabilities.gpus - gpus_needed, n.load))
        if self.policy is SchedulingPolicy.LOCALITY_AWARE and prefer_rack is not None:
            same = [n for n in ok if n.rack == prefer_rack]
            ok = same or ok
        return min(ok, key=lambda n: n.load)


class ClusterManager:
    def __init__(self, config: Optional[ClusterConfig] = None, clock: Callable[[], float] = time.monotonic):
        self.config = config or ClusterConfig()
        self.nodes: Dict[int, NodeInfo] = {}
        self.process_groups: Dict[str, List[int]] = {}
        self.scheduler = ResourceScheduler(self.config.scheduling)
        self.monitor = HeartbeatMonitor(self.nodes, self.config.fault_tolerance, self.handle_node_failure, clock)
        self.events: List[dict] = []
        self.on_group_changed: Optional[Callable[[str, List[int]], None]] = None

    def add_node(self, node: NodeInfo) -> None:
        self.nodes[node.node_id] = node

    def remove_node(self, node_id: int) -> None:
        self.nodes.pop(node_id, None)

    def start(self) -> None:
        if self.config.fault_tolerance.enable_failover:
            self.monitor.start()

    def stop(self) -> None:
        self.monitor.stop()

    def heartbeat(self, node_id: int) -> None:
        self.monitor.beat(node_id)

    def create_process_group(self, name: str, node_ids: List[int]) -> List[int]:
        bad = [n for n in node_ids if n not in self.nodes or self.nodes[n].status is NodeStatus.FAILED]
        if bad:
            raise ValueError(f"nodes {bad} are unknown or failed")
        self.process_groups[name] = list(node_ids)
        return self.process_groups[name]

    def submit_job(self, job: str, gpus: int = 1, prefer_rack: Optional[str] = None) -> Optional[int]:
        n = self.scheduler.select(list(self.nodes.values()), gpus, prefer_rack)
        if n is None:
            return None
        n.jobs.append(job)
        n.load += gpus / max(1, n.capabilities.gpus)
        return n.node_id

    # ---------------------------------------------------------------- failover
    def find_replacement_node(self, failed: NodeInfo) -> Optional[NodeInfo]:
        cands = [n for n in self.nodes.values() if n.node_id != failed.node_id]
        return self.scheduler.select(cands, 1, failed.rack)

    def migrate_jobs(self, src: NodeInfo, dst: NodeInfo) -> List[str]:
        moved, src.jobs = list(src.jobs), []
        dst.jobs.extend(moved)
        dst.load += src.load
        src.load = 0.0
        return moved

    def update_process_groups(self, failed_id: int, replacement_id: Optional[int]) -> Dict[str, List[int]]:
        changed = {}
        for name, members in self.process_groups.items():
            if failed_id in members:
                new = [replacement_id if (m == failed_id and replacement_id is not None and replacement_id not in members)
                       else m for m in members if not (m == failed_id and (replacement_id is None or replacement_id in members))]
                self.process_groups[name] = new
                changed[name] = new
                if self.on_group_changed:
                    self.on_group_changed(name, new)
        return changed

    def handle_node_failure(self, node_id: int) -> dict:
        node = self.nodes[node_id]
        node.status = NodeStatus.FAILED
        ev = {"node": node_id, "time": time.time(), "replacement": None, "migrated": [], "groups": {}}
        if self.config.fault_tolerance.enable_failover:
            rep = self.find_replacement_node(node)
            if rep is not None:
                ev["replacement"] = rep.node_id
                ev["migrated"] = self.migrate_jobs(node, rep)
            ev["groups"] = self.update_process_groups(node_id, rep.node_id if rep else None)
        self.events.append(ev)
        return ev

    trigger_failover = handle_node_failure

    def get_cluster_status(self) -> dict:
        by = {}
        for n in self.nodes.values():
            by[n.status.value] = by.get(n.status.value, 0) + 1
        return {"name": self.config.name, "nodes": len(self.nodes), "by_status": by,
                "groups": {k: list(v) for k, v in self.process_groups.items()}, "failures": len(self.events)}


def retry(fn: Callable, config: FaultToleranceConfig, on_retry: Optional[Callable[[int, BaseException], None]] = None):
    """Call ``fn`` up to ``max_retries`` + 1 times with ``retry_delay`` between attempts."""
    last = None
    for attempt in range(config.max_retries + 1):
        try:
            return fn()
        except Exception as e:  # noqa: BLE001
            last = e
            if on_retry:
                on_retry(attempt, e)
            if attempt < config.max_retries:
                time.sleep(config.retry_delay)
    raise last
