"""Description of the machines a plan is made for (python/paddle/distributed/auto_parallel/static/cluster.py):
``Cluster`` holds machines, their devices and the links between them, is built from a JSON file or generated for a
homogeneous set of nodes, and answers the planner's questions - devices of a type, bandwidth / latency between two
devices, whether a group of ranks crosses machines.

The generated default is an HGX B200 node: eight GPUs with 180 GB each behind an NVSwitch, so that every pair inside
a machine has the same link (type ``NVL``) and the cost of a collective does not depend on which ranks take part,
only on how many.  Between machines the link type is ``NET``.  The figures of the default are measured ones where
this repository has them (copy bandwidth, dense bf16 GEMM rate, bus bandwidth of an 8-rank all-reduce, device-to-device
copy rate) and nominal ones elsewhere."""
from __future__ import annotations

import json
import os
from enum import IntEnum


class DeviceType(IntEnum):
    UNKNOWN = 0
    CPU = 1
    GPU = 2
    XPU = 3
    NPU = 4
    DCU = 5
    NIC = 6


class LinkType(IntEnum):
    UNKNOWN = 0
    LOC = 1
    SYS = 2
    PHB = 3
    PIX = 4
    PIB = 5
    NVL = 6
    NVB = 7
    NET = 8


# rates per device model: half / single / double precision GFLOP/s (dense), memory in GB, link GB/s inside a machine
_MODELS = {
    "B200": dict(hp=1.30e6, sp=8.0e4, dp=4.0e4, memory=180, intra_bw=770.0, hbm=6500.0),
    "H100": dict(hp=7.0e5, sp=6.7e4, dp=3.4e4, memory=80, intra_bw=380.0, hbm=3000.0),
    "A100": dict(hp=2.8e5, sp=1.95e4, dp=9.7e3, memory=80, intra_bw=235.0, hbm=1800.0),
    "V100": dict(hp=1.1e5, sp=1.57e4, dp=7.8e3, memory=32, intra_bw=120.0, hbm=800.0),
}


class Device:
    """One processor of a machine.  ``hp_gflops`` is the dense 16-bit tensor rate."""

    def __init__(self, global_id, local_id, machine):
        self.global_id, self.local_id, self.machine = global_id, local_id, machine
        self.type = DeviceType.UNKNOWN
        self.model = None
        self.dp_gflops = self.sp_gflops = self.hp_gflops = 0.0
        self.memory = 0.0                      # GB
        self.hbm_bandwidth = 0.0               # GB/s
        self._links = {}

    def add_link(self, link):
        self._links[link.target.global_id] = link

    def to_json(self):
        return {"global_id": self.global_id, "local_id": self.local_id, "type": self.type.name, "model": self.model,
                "sp_gflops": self.sp_gflops, "dp_gflops": self.dp_gflops, "hp_gflops": self.hp_gflops,
                "memory": self.memory, "hbm_bandwidth": self.hbm_bandwidth}

    def __repr__(self):
        return f"Device(global_id={self.global_id}, local_id={self.local_id}, machine={self.machine.id}, " \
               f"type={self.type.name}, model={self.model})"

    __str__ = __repr__


class Link:
    """A directed connection between two devices; bandwidth in GB/s, latency in microseconds."""

    def __init__(self, source, target):
        self.source, self.target = source, target
        self.type = LinkType.UNKNOWN
        self.bandwidth = 0.0
        self.latency = 0.0
        self.hop = 1

    def to_json(self):
        return {"source_global_id": self.source.global_id, "target_global_id": self.target.global_id,
                "type": self.type.name, "bandwidth": self.bandwidth, "latency": self.latency}

    def __repr__(self):
        return f"Link({self.source.global_id}->{self.target.global_id}, {self.type.name}, {self.bandwidth} GB/s)"

    __str__ = __repr__


class Machine:
    def __init__(self, id):
        self.id = id
        self.hostname = self.addr = None
        self.port = None
        self.bandwidth = 0.0                   # GB/s of the network interface
        self.latency = 0.0
        self._devices, self._links = {}, {}

    devices = property(lambda self: self._devices)
    links = property(lambda self: self._links)

    @property
    def accelerators(self):
        return {k: d for k, d in self._devices.items() if d.type not in (DeviceType.CPU, DeviceType.NIC)}

    def add_device(self, device):
        self._devices[device.global_id] = device

    def get_device(self, global_id):
        return self._devices.get(global_id)

    def add_link(self, link):
        self._links[(link.source.global_id, link.target.global_id)] = link
        link.source.add_link(link)

    def get_link(self, source_global_id, target_global_id):
        return self._links.get((source_global_id, target_global_id))

    def to_json(self):
        return {"hostname": self.hostname, "addr": self.addr, "port": self.port,
                "devices": [d.to_json() for d in self._devices.values()],
                "links": [l.to_json() for l in self._links.values()]}

    def __repr__(self):
        return f"Machine(id={self.id}, hostname={self.hostname}, devices={len(self._devices)})"


class AlphaLatency:
    """Start-up latencies (microseconds) of collectives by algorithm and scope; missing entries are ``None``."""

    def __init__(self, alpha_latency):
        a = alpha_latency or {}
        self.base_ring = (a.get("base") or {}).get("ring")
        self.base_tree = (a.get("base") or {}).get("tree")
        self.inter_ring = (a.get("inter") or {}).get("ring")
        self.inter_tree = (a.get("inter") or {}).get("tree")
        self.intra_ring = (a.get("intra") or {}).get("ring")
        self.intra_tree = (a.get("intra") or {}).get("tree")
        self.switch = a.get("switch")


class Cluster:
    """Machines, devices and links of a job.  ``gen_default_config_cluster`` writes and loads the description of
    ``node_count`` identical machines; ``build_from_file`` reads one that the user wrote."""

    def __init__(self):
        self._machines = {}
        self._devices = {}
        self._alpha_latency = None
        self._num_devices_per_machine = None
        self.initialized = False

    machines = property(lambda self: self._machines)
    alpha_latency = property(lambda self: self._alpha_latency)

    # ---------------------------------------------------------------- construction
    def gen_default_config_cluster(self, gpu_model="B200", cpu_model="6271C", node_count=1, device_count=8,
                                   gpu_memory=None, cpu_memory=2048, intra_bandwidth=None, inter_bandwidth=50.0,
                                   gpu_dp_gflops=None, gpu_sp_gflops=None, gpu_hp_gflops=None,
                                   cpu_dp_gflops=750.0, cpu_sp_gflops=1500.0, cluster_path=None):
        m = _MODELS.get(gpu_model)
        if m is None:
            raise ValueError(f"unknown gpu model {gpu_model!r}; known: {sorted(_MODELS)}")
        info = {"machines": [], "alpha_latency": {"intra": {"ring": 8.0, "tree": 25.0}, "inter": {"ring": 9.6, "tree": 28.0},
                                                  "base": {"ring": 8.4, "tree": 0.0}, "switch": 10.0}}
        gid = 0
        for n in range(node_count):
            devices = []
            for l in range(device_count):
                devices.append({"global_id": gid, "local_id": l, "type": "GPU", "model": gpu_model,
                                "memory": gpu_memory if gpu_memory is not None else m["memory"],
                                "sp_gflops": gpu_sp_gflops or m["sp"], "dp_gflops": gpu_dp_gflops or m["dp"],
                                "hp_gflops": gpu_hp_gflops or m["hp"], "hbm_bandwidth": m["hbm"]})
                gid += 1
            devices.append({"global_id": gid, "local_id": 0, "type": "CPU", "model": cpu_model, "memory": cpu_memory,
                            "sp_gflops": cpu_sp_gflops, "dp_gflops": cpu_dp_gflops})
            gid += 1
            devices.append({"global_id": gid, "local_id": 0, "type": "NIC", "model": "NET"})
            gid += 1
            info["machines"].append({"hostname": f"host_{n}", "addr": "127.0.0.1", "port": 60009 + n, "devices": devices,
                                     "links": [], "bandwidth": inter_bandwidth})
        bw = intra_bandwidth if intra_bandwidth is not None else m["intra_bw"]
        gpus = [(mi, d["global_id"]) for mi, mach in enumerate(info["machines"]) for d in mach["devices"] if d["type"] == "GPU"]
        for mi, s in gpus:
            for mj, t in gpus:
                if s == t:
                    continue
                same = mi == mj
                info["machines"][mi]["links"].append({"source_global_id": s, "target_global_id": t,
                                                      "type": "NVL" if same else "NET",
                                                      "bandwidth": bw if same else inter_bandwidth,
                                                      "latency": 1.0 if same else 5.0})
        if cluster_path is not None:
            os.makedirs(os.path.dirname(os.path.abspath(cluster_path)), exist_ok=True)
            with open(cluster_path, "w") as f:
                json.dump(info, f, indent=2)
        self._build_from_dict(info)
        return info

    def build_from_file(self, json_file_path):
        with open(json_file_path) as f:
            self._build_from_dict(json.load(f))

    def _build_from_dict(self, info):
        self._machines, self._devices = {}, {}
        for mid, mi in enumerate(info["machines"]):
            mach = Machine(mid)
            mach.hostname, mach.addr, mach.port = mi.get("hostname"), mi.get("addr"), mi.get("port")
            mach.bandwidth, mach.latency = float(mi.get("bandwidth", 0) or 0), float(mi.get("latency", 0) or 0)
            self._machines[mid] = mach
            for di in mi.get("devices", []):
                dev = Device(di["global_id"], di.get("local_id", 0), mach)
                dev.type = DeviceType[di.get("type", "UNKNOWN")]
                dev.model = di.get("model")
                dev.sp_gflops, dev.dp_gflops = float(di.get("sp_gflops", 0) or 0), float(di.get("dp_gflops", 0) or 0)
                dev.hp_gflops = float(di.get("hp_gflops", 0) or 0) or 2 * dev.sp_gflops
                dev.memory = float(di.get("memory", 0) or 0)
                dev.hbm_bandwidth = float(di.get("hbm_bandwidth", 0) or 0) or (_MODELS.get(dev.model or "", {}).get("hbm", 1000.0))
                mach.add_device(dev)
                self._devices[dev.global_id] = dev
        for mid, mi in enumerate(info["machines"]):
            for li in mi.get("links", []):
                s, t = self._devices[li["source_global_id"]], self._devices[li["target_global_id"]]
                link = Link(s, t)
                link.type = LinkType[li.get("type", "UNKNOWN")]
                link.bandwidth, link.latency = float(li.get("bandwidth", 0) or 0), float(li.get("latency", 0) or 0)
                self._machines[mid].add_link(link)
        self._alpha_latency = AlphaLatency(info.get("alpha_latency")) if info.get("alpha_latency") else None
        counts = {len(m.accelerators) for m in self._machines.values()}
        self._num_devices_per_machine = counts.pop() if len(counts) == 1 else None
        self.initialized = True

    # ---------------------------------------------------------------- queries
    def get_all_devices(self, device_type="GPU"):
        t = DeviceType[device_type] if isinstance(device_type, str) else device_type
        return [d for d in self._devices.values() if d.type == t]

    def get_device(self, global_id):
        return self._devices[global_id]

    def get_num_machines(self):
        return len(self._machines)

    def get_num_devices_per_machine(self):
        return self._num_devices_per_machine

    def _rank_device(self, rank):
        """Ranks number the accelerators in order of their global ids."""
        gpus = sorted(d.global_id for d in self._devices.values() if d.type not in (DeviceType.CPU, DeviceType.NIC))
        return self._devices[gpus[rank]]

    def get_beta(self, source_rank, target_rank):
        """Seconds per byte between two ranks (the reference returns microseconds per megabyte-ish units of its own; the
        cost classes here work in seconds and bytes throughout)."""
        if source_rank == target_rank:
            return 0.0
        s, t = self._rank_device(source_rank), self._rank_device(target_rank)
        link = s.machine.get_link(s.global_id, t.global_id)
        bw = link.bandwidth if link is not None and link.bandwidth > 0 else (s.machine.bandwidth or 10.0)
        return 1.0 / (bw * 1e9)

    def get_latency(self, source_rank, target_rank):
        s, t = self._rank_device(source_rank), self._rank_device(target_rank)
        link = s.machine.get_link(s.global_id, t.global_id)
        return (link.latency if link is not None else 5.0) * 1e-6

    def cross_machine(self, ranks):
        return len({self._rank_device(r).machine.id for r in ranks}) > 1

    def get_involved_machine_count(self, ranks):
        return len({self._rank_device(r).machine.id for r in ranks})

    def convert_rank_to_device_id(self, rank):
        return self._rank_device(rank).global_id

    def get_hop(self, source_rank, target_rank):
        return 0 if source_rank == target_rank else (2 if self.cross_machine([source_rank, target_rank]) else 1)

    def to_json(self):
        return {"machines": [m.to_json() for m in self._machines.values()]}

    def __repr__(self):
        return f"Cluster(machines={len(self._machines)}, accelerators={len(self.get_all_devices('GPU'))})"


def get_default_cluster(json_config=None, node_count=None, device_count=None):
    """The cluster of the running job: from ``json_config["cluster"]`` (a ``path`` to a description or ``num_nodes`` /
    ``num_gpus`` / ``gpu_model`` / ``gpu_memory``), else from the launcher's environment, else one B200 node."""
    cluster = Cluster()
    cfg = (json_config or {}).get("cluster") if isinstance(json_config, dict) else None
    if cfg and "path" in cfg:
        cluster.build_from_file(cfg["path"])
        return cluster
    if cfg:
        for k in ("num_nodes", "num_gpus", "gpu_model", "gpu_memory"):
            if k not in cfg:
                raise ValueError(f"the cluster section needs {k!r} when it gives no path")
        cluster.gen_default_config_cluster(gpu_model=cfg["gpu_model"], node_count=cfg["num_nodes"],
                                           device_count=cfg["num_gpus"], gpu_memory=cfg["gpu_memory"])
        return cluster
    if node_count is None:
        node_count = int(os.environ.get("PADDLE_TRAINERS_NUM", os.environ.get("NNODES", "1")) or 1)
    if device_count is None:
        world = int(os.environ.get("PADDLE_GLOBAL_SIZE", os.environ.get("WORLD_SIZE", "0")) or 0)
        local = int(os.environ.get("PADDLE_LOCAL_SIZE", os.environ.get("LOCAL_WORLD_SIZE", "0")) or 0)
        device_count = local or (world // node_count if world else 8)
    cluster.gen_default_config_cluster(node_count=node_count, device_count=device_count)
    return cluster
