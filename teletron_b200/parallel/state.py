"""Process topology and groups: TP x CP x DP (x PP) inside a DiT replica, several replicas
("consumer models") and encoder ("producer") ranks appended after the DiT ranks.

``Topology`` is pure arithmetic (unit-testable without torch.distributed).  It reproduces the
reference layout (teletron/core/parallel_state.py:156-642): inside a replica TP varies fastest,
then CP, then DP, then PP; replica k owns ranks [k*W, (k+1)*W); the last
``encoder_ranks`` ranks of the world only run encoders; the TP x CP leader of DP rank i is fed
by producer ``dit_world + i % encoder_ranks`` (parallel_state.py:274-290).
``initialize_model_parallel`` builds the torch.distributed groups (NCCL on GPU, gloo on CPU)
and the getters mirror Megatron's names so user code ports directly.  Instead of
monkey-patching ``torch.distributed`` defaults (parallel_state.py:37-154) callers pass
``get_transformer_model_group()`` explicitly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class CommPair:
    producer: int
    consumer: int
    dp_rank: int
    dp_size: int


@dataclass(frozen=True)
class Topology:
    world_size: int
    tp: int = 1
    cp: int = 1
    pp: int = 1
    encoder_ranks: int = 0
    replicas: int = 1
    ep: int = 1

    def __post_init__(self):
        dit = self.world_size - self.encoder_ranks
        if dit <= 0:
            raise ValueError("no DiT ranks left after reserving encoder ranks")
        if dit % self.replicas:
            raise ValueError(f"DiT world {dit} not divisible by {self.replicas} replicas")
        per = dit // self.replicas
        mp = self.tp * self.cp * self.pp
        if per % mp:
            raise ValueError(f"replica world {per} not divisible by tp*cp*pp = {mp}")
        if (per // mp) % self.ep:
            raise ValueError(f"data-parallel size {per // mp} not divisible by the expert-parallel size {self.ep}")

    # ---- sizes
    @property
    def dit_world(self) -> int:
        return self.world_size - self.encoder_ranks

    @property
    def replica_world(self) -> int:
        return self.dit_world // self.replicas

    @property
    def dp(self) -> int:
        return self.replica_world // (self.tp * self.cp * self.pp)

    # ---- rank <-> coordinates
    def is_encoder_rank(self, rank: int) -> bool:
        return rank >= self.dit_world

    def coords(self, rank: int) -> Dict[str, int]:
        if self.is_encoder_rank(rank):
            return dict(encoder=rank - self.dit_world)
        rep, r = divmod(rank, self.replica_world)
        tp_i = r % self.tp
        cp_i = (r // self.tp) % self.cp
        dp_i = (r // (self.tp * self.cp)) % self.dp
        pp_i = r // (self.tp * self.cp * self.dp)
        return dict(replica=rep, pp=pp_i, dp=dp_i, cp=cp_i, tp=tp_i)

    def rank_of(self, replica=0, pp=0, dp=0, cp=0, tp=0) -> int:
        return (replica * self.replica_world + pp * (self.dp * self.cp * self.tp) +
                dp * (self.cp * self.tp) + cp * self.tp + tp)

    # ---- group enumerations (each a list of rank lists, identical on every rank)
    def _groups(self, vary: List[str]) -> List[List[int]]:
        sizes = dict(pp=self.pp, dp=self.dp, cp=self.cp, tp=self.tp)
        fixed = [k for k in ("pp", "dp", "cp", "tp") if k not in vary]
        out = []
        for rep in range(self.replicas):
            def rec(idx, cur):
                if idx == len(fixed):
                    members = []

                    def rec2(j, c2):
                        if j == len(vary):
                            members.append(self.rank_of(replica=rep, **c2))
                            return
                        for v in range(sizes[vary[j]]):
                            rec2(j + 1, {**c2, vary[j]: v})

                    rec2(0, dict(cur))
                    out.append(sorted(members))
                    return
                for v in range(sizes[fixed[idx]]):
                    rec(idx + 1, {**cur, fixed[idx]: v})

            rec(0, {})
        return out

    def tp_groups(self): return self._groups(["tp"])
    def cp_groups(self): return self._groups(["cp"])
    def pp_groups(self): return self._groups(["pp"])
    def dp_groups(self, with_cp: bool = False): return self._groups(["dp", "cp"] if with_cp else ["dp"])
    def tp_cp_groups(self): return self._groups(["cp", "tp"])
    def model_parallel_groups(self): return self._groups(["pp", "cp", "tp"]) if self.cp > 1 else self._groups(["pp", "tp"])
    def replica_groups(self): return [list(range(k * self.replica_world, (k + 1) * self.replica_world)) for k in range(self.replicas)]
    def dit_group(self): return list(range(self.dit_world))

    # expert parallelism lives inside data parallelism (teletron/core/parallel_state.py:596-633): `ep` consecutive
    # data-parallel ranks hold different experts; ranks with the same expert form the "data modulo expert" group
    def ep_groups(self) -> List[List[int]]:
        out = []
        for g in self._groups(["dp"]):
            out.extend(g[i:i + self.ep] for i in range(0, len(g), self.ep))
        return out

    def tp_ep_groups(self) -> List[List[int]]:
        out = []
        for g in self._groups(["dp", "tp"]):          # sorted: tp fastest inside each dp index
            n = self.ep * self.tp
            out.extend(g[i:i + n] for i in range(0, len(g), n))
        return out

    def dp_modulo_ep_groups(self) -> List[List[int]]:
        out = []
        for g in self._groups(["dp"]):
            out.extend(g[j::self.ep] for j in range(self.ep))
        return out

    # first and last pipeline stage share the embedding weights' gradients; the first stage alone holds position
    # embeddings (parallel_state.py:495-542).  With one stage both groups are the rank itself.
    def embedding_groups(self) -> List[List[int]]:
        return [sorted({g[0], g[-1]}) for g in self.pp_groups()]

    def position_embedding_groups(self) -> List[List[int]]:
        return [[g[0]] for g in self.pp_groups()]

    def tp_cp_leaders(self) -> List[int]:
        return [g[0] for g in self.tp_cp_groups()]

    def comm_pairs(self) -> List[CommPair]:
        """One pair per TP x CP leader: which encoder rank feeds it and which data shard it reads."""
        if self.encoder_ranks == 0:
            return []
        pairs = []
        for i, leader in enumerate(self.tp_cp_leaders()):
            c = self.coords(leader)
            pairs.append(CommPair(producer=self.dit_world + i % self.encoder_ranks, consumer=leader,
                                  dp_rank=c["dp"], dp_size=self.dp))
        return pairs


class _State:
    topo: Optional[Topology] = None
    rank: int = 0
    groups: Dict[str, object] = {}
    ranks: Dict[str, List[int]] = {}
    gloo: Dict[str, object] = {}


_S = _State()


def _new_groups(name: str, rank_lists: List[List[int]], rank: int, backend=None, timeout=None, gloo_twin=False):
    for rl in rank_lists:
        kw = {}
        if timeout is not None:
            kw["timeout"] = timeout
        g = dist.new_group(rl, backend=backend, **kw)
        tw = dist.new_group(rl, backend="gloo", **kw) if gloo_twin else None
        if rank in rl:
            _S.groups[name] = g
            _S.ranks[name] = rl
            if tw is not None:
                _S.gloo[name] = tw


def initialize_model_parallel(tensor_model_parallel_size: int = 1, pipeline_model_parallel_size: int = 1,
                              context_parallel_size: int = 1, encoder_world_size: int = 0,
                              consumer_models_num: int = 1, timeout=None, gloo_twins: bool = False,
                              expert_model_parallel_size: int = 1) -> Topology:
    """Create every process group. Must be called by all ranks of the world (encoder ranks too)."""
    assert dist.is_initialized(), "call torch.distributed.init_process_group first"
    world, rank = dist.get_world_size(), dist.get_rank()
    topo = Topology(world, tensor_model_parallel_size, context_parallel_size, pipeline_model_parallel_size,
                    encoder_world_size, consumer_models_num, expert_model_parallel_size)
    _S.topo, _S.rank = topo, rank
    _S.groups, _S.ranks, _S.gloo = {}, {}, {}
    _S.groups["world"] = dist.group.WORLD
    _S.ranks["world"] = list(range(world))
    _new_groups("dit", [topo.dit_group()], rank, timeout=timeout)
    _new_groups("replica", topo.replica_groups(), rank, timeout=timeout)
    _new_groups("tp", topo.tp_groups(), rank, timeout=timeout)
    _new_groups("cp", topo.cp_groups(), rank, timeout=timeout)
    _new_groups("pp", topo.pp_groups(), rank, timeout=timeout)
    _new_groups("dp", topo.dp_groups(False), rank, timeout=timeout, gloo_twin=gloo_twins)
    _new_groups("dp_cp", topo.dp_groups(True), rank, timeout=timeout, gloo_twin=gloo_twins)
    _new_groups("tp_cp", topo.tp_cp_groups(), rank, timeout=timeout)
    _new_groups("mp", topo.model_parallel_groups(), rank, timeout=timeout)
    _new_groups("embd", topo.embedding_groups(), rank, timeout=timeout)
    _new_groups("pos_embd", topo.position_embedding_groups(), rank, timeout=timeout)
    if topo.ep > 1:
        _new_groups("ep", topo.ep_groups(), rank, timeout=timeout)
        _new_groups("tp_ep", topo.tp_ep_groups(), rank, timeout=timeout)
        _new_groups("dp_mod_ep", topo.dp_modulo_ep_groups(), rank, timeout=timeout, gloo_twin=gloo_twins)
    return topo


def destroy_model_parallel():
    _S.topo = None
    _S.groups, _S.ranks, _S.gloo = {}, {}, {}


def warm_up_groups(names=None) -> None:
    """Creates the communicators of groups whose first collective comes late, now, with one tiny all-reduce each.

    NCCL builds a group's communicator at the group's first collective and allocates its buffers with the driver's
    own allocator.  The groups of the training step itself meet theirs in the first step; the group of all
    transformer ranks is first used by the timer summary of the first log line, when the caching allocator may
    already hold every free byte of a large model's GPU, and the communicator then fails with an out-of-memory error
    that no amount of cached memory can satisfy.  ``names`` defaults to that group and the data x context parallel one.  Groups of one rank and groups
    this rank is not part of are skipped; every rank walks the names in the same order, and groups of one kind are
    disjoint, so the collectives pair up."""
    if _S.topo is None or not dist.is_initialized():
        return
    if names is None:
        # ... and the data x context parallel group: with the peer-memory optimizer its first NCCL use may be the
        # gather of the optimizer state at the first checkpoint
        names = ("replica" if _S.topo.replicas > 1 else "dit", "dp_cp")
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    for name in names:
        g = _S.groups.get(name)
        if g is None or len(_S.ranks.get(name, ())) <= 1:
            continue
        dist.all_reduce(torch.zeros(1, device=dev), group=g)
    if dev == "cuda":
        torch.cuda.synchronize()


def model_parallel_is_initialized() -> bool:
    return _S.topo is not None


def get_topology() -> Topology:
    assert _S.topo is not None, "model parallel state is not initialised"
    return _S.topo


def _group(name):
    if _S.topo is None:
        return None
    return _S.groups.get(name)


def _size(name):
    return len(_S.ranks[name]) if (_S.topo is not None and name in _S.ranks) else 1


def _rank_in(name):
    return _S.ranks[name].index(_S.rank) if (_S.topo is not None and name in _S.ranks) else 0


def is_encoder_rank() -> bool:
    return _S.topo is not None and _S.topo.is_encoder_rank(_S.rank)


def get_world_group(): return _group("world")
def get_transformer_model_group(): return _group("replica") if (_S.topo and _S.topo.replicas > 1) else _group("dit")
def get_tensor_model_parallel_group(): return _group("tp")
def get_tensor_model_parallel_world_size(): return _size("tp")
def get_tensor_model_parallel_rank(): return _rank_in("tp")
def get_context_parallel_group(): return _group("cp")
def get_context_parallel_world_size(): return _size("cp")
def get_context_parallel_rank(): return _rank_in("cp")
def get_pipeline_model_parallel_group(): return _group("pp")
def get_pipeline_model_parallel_world_size(): return _size("pp")
def get_model_parallel_group(): return _group("mp")
def get_data_parallel_group(with_context_parallel: bool = False): return _group("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_group_gloo(with_context_parallel: bool = False): return _S.gloo.get("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_world_size(with_context_parallel: bool = False): return _size("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_rank(with_context_parallel: bool = False): return _rank_in("dp_cp" if with_context_parallel else "dp")
def get_tensor_context_parallel_group(): return _group("tp_cp")
def get_tensor_context_parallel_world_size(): return _size("tp_cp")
def get_tensor_context_parallel_rank(): return _rank_in("tp_cp")
def get_tensor_context_parallel_src_rank(): return _S.ranks["tp_cp"][0] if (_S.topo and "tp_cp" in _S.ranks) else 0
def get_embedding_group(): return _group("embd")
def get_position_embedding_group(): return _group("pos_embd")
def is_rank_in_embedding_group(): return _S.topo is not None and _S.rank in _S.ranks.get("embd", [])
def get_expert_model_parallel_group(): return _group("ep")
def get_expert_model_parallel_world_size(): return _size("ep")
def get_expert_model_parallel_rank(): return _rank_in("ep")
def get_tensor_and_expert_parallel_group(): return _group("tp_ep")
def get_data_modulo_expert_parallel_group(): return _group("dp_mod_ep")
def get_data_modulo_expert_parallel_rank(): return _rank_in("dp_mod_ep")
def get_group_ranks(name: str) -> List[int]: return list(_S.ranks.get(name, [0]))


def get_comm_pair() -> List[CommPair]:
    """Pairs this rank takes part in: a producer gets all its consumers, a TP x CP leader its one pair."""
    if _S.topo is None:
        return []
    return [p for p in _S.topo.comm_pairs() if _S.rank in (p.producer, p.consumer)]
