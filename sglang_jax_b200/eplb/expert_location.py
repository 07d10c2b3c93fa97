"""Logical -> physical expert placement with redundancy (reference
`python/sgl_jax/srt/eplb/expert_location.py`, `eplb_algorithms/deepseek.py`).

`ExpertLocation` maps each logical expert to one or more physical slots spread over the EP
ranks; the router's ids are rewritten to physical slots (replicas picked round-robin by token) so
hot experts are served by several GPUs.  `rebalance` implements the DeepSeek EPLB heuristic:
replicate the heaviest experts, then pack physical experts onto ranks greedily by load;
`rebalance_hierarchical` is its node-aware form for group-limited routing."""

from __future__ import annotations

import csv
import os
import time

import numpy as np
import torch


def replicate_experts(weight: np.ndarray, num_phy: int) -> tuple[np.ndarray, np.ndarray]:
    """Give the `num_phy - num_logical` spare slots to the experts with the highest load per replica.
    Returns (phy2log [num_phy], replica_count [num_logical])."""
    n = len(weight)
    assert num_phy >= n
    phy2log = list(range(n))
    cnt = np.ones(n, dtype=np.int64)
    for _ in range(num_phy - n):
        e = int(np.argmax(weight / cnt))
        phy2log.append(e)
        cnt[e] += 1
    return np.asarray(phy2log, dtype=np.int64), cnt


def balanced_packing(weight: np.ndarray, num_packs: int) -> np.ndarray:
    """Assign items to `num_packs` equal-size packs, heaviest first into the lightest pack.
    Returns pack index per item."""
    n = len(weight)
    assert n % num_packs == 0
    cap = n // num_packs
    order = np.argsort(-weight, kind="stable")
    load = np.zeros(num_packs)
    fill = np.zeros(num_packs, dtype=np.int64)
    out = np.empty(n, dtype=np.int64)
    for i in order:
        cand = [p for p in range(num_packs) if fill[p] < cap]
        p = min(cand, key=lambda q: (load[q], q))
        out[i] = p
        load[p] += weight[i]
        fill[p] += 1
    return out


def rebalance(expert_load: np.ndarray, num_phy: int, num_ranks: int) -> np.ndarray:
    """phy2log of length `num_phy`, ordered so that rank r owns slots [r*S, (r+1)*S)."""
    phy2log, cnt = replicate_experts(expert_load.astype(np.float64), num_phy)
    per_replica = expert_load[phy2log] / cnt[phy2log]
    pack = balanced_packing(per_replica, num_ranks)
    order = np.argsort(pack, kind="stable")
    return phy2log[order]


def rebalance_hierarchical(expert_load: np.ndarray, num_phy: int, num_groups: int, num_nodes: int,
                           num_ranks: int) -> np.ndarray:
    """Placement for group-limited routing across several nodes (reference `eplb_algorithms/deepseek.py`
    `rebalance_experts_hierarchical`): (1) whole expert groups are packed onto nodes so that the groups a token may
    choose from sit on one node, (2) inside every node the spare slots go to its experts with the highest load per
    replica, (3) the node's physical experts are packed onto its ranks.  Returns phy2log of length `num_phy`, rank r
    owning slots `[r * S, (r + 1) * S)`, ranks `[n * R, (n + 1) * R)` forming node n."""
    load = np.asarray(expert_load, dtype=np.float64)
    E = len(load)
    if num_groups % num_nodes or E % num_groups or num_ranks % num_nodes or num_phy % num_ranks:
        raise ValueError(f"groups ({num_groups}) must divide over nodes ({num_nodes}), experts ({E}) over groups, "
                         f"ranks ({num_ranks}) over nodes and physical experts ({num_phy}) over ranks")
    gsize = E // num_groups
    group_node = balanced_packing(load.reshape(num_groups, gsize).sum(1), num_nodes)
    phy_per_node, ranks_per_node = num_phy // num_nodes, num_ranks // num_nodes
    out = []
    for node in range(num_nodes):
        experts = np.concatenate([np.arange(g * gsize, (g + 1) * gsize) for g in np.nonzero(group_node == node)[0]])
        local, cnt = replicate_experts(load[experts], phy_per_node)
        pack = balanced_packing(load[experts][local] / cnt[local], ranks_per_node)
        out.append(experts[local[np.argsort(pack, kind="stable")]])
    return np.concatenate(out).astype(np.int64)


def rebalance_experts(expert_load: np.ndarray, num_phy: int, num_ranks: int, num_groups: int = 1, num_nodes: int = 1,
                      algorithm: str = "auto") -> np.ndarray:
    """One layer's phy2log.  `algorithm`: `deepseek` (global), `deepseek_hierarchical`, or `auto`, which takes the
    hierarchical form when the groups divide over the nodes (reference `eplb_algorithms/__init__.py`
    `compute_algorithm`)."""
    if algorithm == "auto":
        algorithm = "deepseek_hierarchical" if num_nodes > 1 and num_groups > 1 and num_groups % num_nodes == 0 \
            else "deepseek"
    if algorithm == "deepseek_hierarchical":
        return rebalance_hierarchical(expert_load, num_phy, num_groups, num_nodes, num_ranks)
    if algorithm != "deepseek":
        raise ValueError(f"unknown EPLB algorithm {algorithm!r}")
    return rebalance(np.asarray(expert_load, dtype=np.float64), num_phy, num_ranks)


class ExpertLocation:
    def __init__(self, num_logical: int, ep_size: int, num_redundant: int = 0, phy2log: np.ndarray | None = None,
                 device="cpu"):
        self.num_logical = num_logical
        self.num_physical = num_logical + num_redundant
        assert self.num_physical % ep_size == 0
        self.ep_size = ep_size
        if phy2log is None:     # "trivial": spares replicate experts 0, 1, 2, ...
            phy2log = np.concatenate([np.arange(num_logical), np.arange(num_redundant) % num_logical])
        self.set_mapping(np.asarray(phy2log, dtype=np.int64), device)

    def set_mapping(self, phy2log: np.ndarray, device="cpu"):
        self.phy2log = phy2log
        reps = [[] for _ in range(self.num_logical)]
        for p, l in enumerate(phy2log):
            reps[int(l)].append(p)
        self.max_rep = max(len(r) for r in reps)
        table = np.full((self.num_logical, self.max_rep), -1, dtype=np.int64)
        for l, r in enumerate(reps):
            assert r, f"logical expert {l} has no physical slot"
            table[l, : len(r)] = r
        self.log2phy = torch.as_tensor(table, device=device)
        self.rep_count = torch.as_tensor([len(r) for r in reps], device=device)

    # `--ep-dispatch-algorithm` (reference `expert_location.py:338-392`): `static` sends every token of a logical
    # expert to its first physical slot, `dynamic` (the default here) deals the tokens over the replicas
    dispatch_algorithm = "dynamic"

    def logical_to_physical(self, topk_ids: torch.Tensor) -> torch.Tensor:
        ids = topk_ids.long()
        if self.log2phy.device != ids.device:
            self.log2phy = self.log2phy.to(ids.device)
            self.rep_count = self.rep_count.to(ids.device)
        if self.dispatch_algorithm == "static":
            return self.log2phy[ids, 0].to(topk_ids.dtype)
        tok = torch.arange(ids.shape[0], device=ids.device).view(-1, 1)
        pick = tok % self.rep_count[ids]
        return self.log2phy[ids, pick].to(topk_ids.dtype)

    def physical_weights(self, logical_weights: torch.Tensor) -> torch.Tensor:
        """Gather `[num_logical, ...]` expert weights into physical slot order."""
        return logical_weights[torch.as_tensor(self.phy2log, device=logical_weights.device)]

    @classmethod
    def from_load(cls, expert_load, ep_size: int, num_redundant: int, device="cpu", num_groups: int = 1,
                  num_nodes: int = 1, algorithm: str = "auto") -> "ExpertLocation":
        load = np.asarray(expert_load, dtype=np.float64)
        phy2log = rebalance_experts(load, len(load) + num_redundant, ep_size, num_groups, num_nodes, algorithm)
        return cls(len(load), ep_size, num_redundant, phy2log, device)


class ExpertDistributionRecorder:
    """Per-layer expert hit counts (`--enable-expert-distribution-recorder`; reference flags
    `expert_distribution_recorder_buffer_size` / `_output_file`).  Counting happens on the device with a
    scatter-add (no synchronisation inside the forward); every `buffer_size` recorded forwards, and at
    shutdown, the totals are written to the output file as a `[layers, experts]` array that
    `--init-expert-location <file>` and `eplb/tools.py` read back."""

    def __init__(self, num_layers: int, num_experts: int, buffer_size: int = 100, output_file: str | None = None,
                 device="cpu"):
        self.counts = torch.zeros((num_layers, num_experts), dtype=torch.int64, device=device)
        self.buffer_size = max(int(buffer_size), 1)
        self.output_file = output_file
        self.forwards = 0
        # kept for callers that used the host ring of the first version
        self.buf = np.zeros((1, num_layers, num_experts), dtype=np.int64)

    def record(self, layer_id: int, topk_ids: torch.Tensor):
        ids = topk_ids.reshape(-1).long()
        if ids.device != self.counts.device:
            ids = ids.to(self.counts.device)
        self.counts[layer_id].scatter_add_(0, ids.clamp_(0, self.counts.shape[1] - 1), torch.ones_like(ids))

    def step(self):
        self.forwards += 1
        if self.forwards % self.buffer_size == 0:
            self.dump()

    def aggregate(self) -> np.ndarray:
        return self.counts.cpu().numpy()

    def dump(self):
        if self.output_file:
            np.save(self.output_file, self.aggregate())


class ExpertBalanceAnalyzer(ExpertDistributionRecorder):
    """`--enable-expert-balance-debug`: the recorder's per-layer hit counts, cut into segments of
    `--expert-balance-segment-counter` decode steps; at the end of a segment one CSV row per layer goes to
    `--expert-balance-output-file` with the counts and, when the experts divide over the expert-parallel ranks, how far
    the busiest rank is above the mean (reference `layers/routed_experts_capturer.py` `_ExpertBalanceAnalyzer`)."""

    HEADER = ["timestamp", "segment_idx", "segment_counter", "segment_decode_steps", "layer", "num_experts", "topk",
              "ep_size", "total_assignments", "max_over_mean_expert", "max_over_mean_device", "experts_count"]

    def __init__(self, num_layers: int, num_experts: int, topk: int, ep_size: int, segment_counter: int = 100,
                 output_file: str | None = None, device="cpu"):
        super().__init__(num_layers, num_experts, buffer_size=1 << 30, output_file=None, device=device)
        self.topk, self.ep_size = int(topk), int(ep_size)
        self.segment_counter = max(int(segment_counter), 1)
        self.csv_file = output_file
        self.segment_idx = 0
        self.decode_steps = 0
        if output_file:
            os.makedirs(os.path.dirname(os.path.abspath(output_file)), exist_ok=True)
            if not os.path.exists(output_file) or os.path.getsize(output_file) == 0:
                with open(output_file, "w", newline="") as f:
                    csv.writer(f).writerow(self.HEADER)

    def step(self, is_decode: bool = True):
        self.forwards += 1
        if not is_decode:
            return
        self.decode_steps += 1
        if self.decode_steps >= self.segment_counter:
            self.flush_segment()

    def flush_segment(self):
        counts = self.aggregate().copy()          # on CPU the array shares the tensor's memory
        self.counts.zero_()
        steps, self.decode_steps = self.decode_steps, 0
        if self.csv_file and counts.sum() > 0:
            now = time.strftime("%Y-%m-%dT%H:%M:%S")
            E = counts.shape[1]
            with open(self.csv_file, "a", newline="") as f:
                w = csv.writer(f)
                for layer, c in enumerate(counts):
                    if c.sum() == 0:
                        continue
                    dev = ""
                    if self.ep_size > 0 and E % self.ep_size == 0:
                        per_dev = c.reshape(self.ep_size, -1).sum(1)
                        dev = round(float(per_dev.max() / max(per_dev.mean(), 1e-9)), 4)
                    w.writerow([now, self.segment_idx, self.segment_counter, steps, layer, E, self.topk, self.ep_size,
                                int(c.sum()), round(float(c.max() / max(c.mean(), 1e-9)), 4), dev,
                                " ".join(map(str, c.tolist()))])
        self.segment_idx += 1


def load_expert_load(path: str) -> np.ndarray:
    """`[layers, experts]` hit counts from a recorder dump (`.npy`) or a JSON list of lists."""
    if path.endswith(".json"):
        import json
        with open(path) as f:
            return np.asarray(json.load(f), dtype=np.float64)
    return np.asarray(np.load(path), dtype=np.float64)
