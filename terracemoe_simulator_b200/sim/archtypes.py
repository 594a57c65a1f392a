"""Plain descriptions the co-design layer works on: an MoE architecture, a two-level fabric, a
machine (accelerator + fabric + arrival-chain tier) and a memory profile.  No pricing happens
here; ``sim/codesign.py`` prices them and re-exports these names.

``Fabric`` carries two bandwidth levels, the fixed cost of one exchange as measured points over
the number of peers (read by clamped linear interpolation) and a half-performance message size;
``levels()`` turns it into the three ``core.Level`` objects the call model wants.

Field lists follow the reference's ``sim/codesign.py`` (``MoEArch`` :56-103, ``Fabric``
:106-150, ``Machine`` :153-173, ``MemoryProfile`` / ``UNMEASURED`` :229-262).
"""
from __future__ import annotations

from dataclasses import dataclass

from .compute import PEAK_TFLOPS, ThroughputCurve
from .core import Level
from .machine import PYTORCH_CHAIN, Accelerator, ArrivalChain


@dataclass(frozen=True)
class MoEArch:
    name: str
    hidden: int
    d_expert: int
    n_experts: int
    k: int
    M: int = 1
    n_shared_experts: int = 0
    n_moe_layers: int = 1
    seq: int = 4096
    mbs: int = 1
    gbs: int = 512
    n_mats: int = 3
    bytes_per_elem: int = 2
    optimizer_bytes_per_param: float = 6.0

    @property
    def q(self) -> int:
        quota, rest = divmod(self.k, self.M)
        if rest:
            raise ValueError("%s: k=%d is not divisible by M=%d, so the per-group quota k/M is "
                             "not an integer" % (self.name, self.k, self.M))
        return quota

    @property
    def tokens_per_rank(self) -> int:
        return self.seq * self.mbs

    def params_per_expert(self) -> int:
        return self.n_mats * self.hidden * self.d_expert

    def expert_bytes_all_layers(self, with_optimizer: bool = True) -> float:
        bytes_per_param = self.bytes_per_elem + with_optimizer * self.optimizer_bytes_per_param
        experts = (self.n_experts + self.n_shared_experts) * self.n_moe_layers
        return experts * self.params_per_expert() * bytes_per_param


@dataclass(frozen=True)
class Fabric:
    name: str
    cards_per_node: int
    nodes: int
    beta_intra_gbps: float
    beta_inter_gbps: float
    alpha_ms: tuple                     # ((world, ms), ...)
    x_half_bytes: float = 0.0

    @property
    def ep(self) -> int:
        return self.cards_per_node * self.nodes

    @property
    def ratio(self) -> float:
        return self.beta_intra_gbps / self.beta_inter_gbps

    def alpha_at(self, world: int) -> float:
        """Fixed cost of one exchange among ``world`` peers: the measured points, interpolated
        linearly and held constant outside their range."""
        return ThroughputCurve(self.alpha_ms)(world)

    def fixed_cost_condition(self) -> dict:
        split = self.alpha_at(self.nodes) + self.alpha_at(self.cards_per_node)
        whole = self.alpha_at(self.ep)
        return {"two_hop_alpha_ms": split, "one_hop_alpha_ms": whole, "clears": split < whole,
                "margin_ms": whole - split}

    def levels(self) -> dict:
        """The three ``core.Level`` objects of this fabric (one-hop sees the slow side)."""
        from .calibrate import saturating_beta
        fixed = sorted(self.alpha_ms)
        curve = {"fast": saturating_beta(self.beta_intra_gbps, self.x_half_bytes),
                 "slow": saturating_beta(self.beta_inter_gbps, self.x_half_bytes)}
        curve["flat"] = curve["slow"]
        return {name: Level(name, fixed, pts) for name, pts in curve.items()}


@dataclass(frozen=True)
class Machine:
    accel: Accelerator
    fabric: Fabric
    chain: ArrivalChain = PYTORCH_CHAIN

    @property
    def transfers_compute(self) -> bool:
        """Does the accelerator bring its own peak, or is platform A's roofline borrowed?"""
        return bool(self.accel.peak_tflops)

    @property
    def peak_tflops(self) -> float:
        return self.accel.peak_tflops if self.transfers_compute else PEAK_TFLOPS

    @property
    def balance_flops_per_byte(self) -> float:
        return self.peak_tflops * 1e3 / self.accel.hbm_gbps


@dataclass(frozen=True)
class MemoryProfile:
    name: str
    activation_bytes_per_token_layer: float
    overhead_frac: float
    recompute: str = "unknown"
    measured: bool = False
    source: str = ""

    def provenance(self) -> str:
        return ("measured: " if self.measured else "ASSUMED: ") + self.source


UNMEASURED = MemoryProfile(name="unmeasured placeholder", activation_bytes_per_token_layer=0.0,
                           overhead_frac=0.15, recompute="assumed full recompute", measured=False,
                           source="invented; a residency measurement protocol would replace it")
