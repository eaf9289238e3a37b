"""Memory and link probe of the visible GPUs, read-only.

The reference probes VRAM and PCIe BAR sizes of its cards before it plans buffers
(src/runtime/vram_bars.h, vram_bars.cc: whether the whole VRAM is host-visible through a resizable BAR).
Here the questions are: how much HBM is free on each GPU (the memory planner's input), how large the
BAR1 aperture is (pinned-host <-> device copies of the prefix store do not need it, mapped access does), and
whether every pair of GPUs of a multi-GPU placement is connected by NVLink (the fused collective kernels store
into peer memory; over PCIe they would work and crawl).

Everything goes through NVML queries (``nvmlDeviceGet*``); nothing is set.  ``probe(nvml=...)`` takes any
object with the NVML functions used here, which is how the tests run it without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

NVLINK_MAX_LINKS = 18


@dataclass
class GpuMemory:
    index: int
    name: str
    total: int
    free: int
    bar1_total: int
    bar1_free: int
    nvlinks_up: int
    peers_nvlink: Dict[int, bool] = field(default_factory=dict)   # other GPU index -> connected by NVLink

    @property
    def bar1_covers_memory(self) -> bool:
        """True when the whole device memory is host-visible through BAR1 (a resizable BAR)."""
        return self.bar1_total >= self.total


def _text(x) -> str:
    return x.decode() if isinstance(x, (bytes, bytearray)) else str(x)


def probe(nvml=None, indices: Optional[List[int]] = None) -> List[GpuMemory]:
    """One ``GpuMemory`` per visible GPU (or per index in ``indices``)."""
    own = nvml is None
    if own:
        import pynvml as nvml   # nvidia-ml-py
        nvml.nvmlInit()
    try:
        n = nvml.nvmlDeviceGetCount()
        idx = list(range(n)) if indices is None else [i for i in indices if 0 <= i < n]
        handles = {i: nvml.nvmlDeviceGetHandleByIndex(i) for i in idx}
        out = []
        for i in idx:
            h = handles[i]
            mem = nvml.nvmlDeviceGetMemoryInfo(h)
            try:
                bar = nvml.nvmlDeviceGetBAR1MemoryInfo(h)
                bar_total, bar_free = int(bar.bar1Total), int(bar.bar1Free)
            except Exception:  # noqa: BLE001   (not reported inside some containers)
                bar_total = bar_free = 0
            links = 0
            for link in range(NVLINK_MAX_LINKS):
                try:
                    if nvml.nvmlDeviceGetNvLinkState(h, link):
                        links += 1
                except Exception:  # noqa: BLE001   (link index beyond the device's links)
                    break
            peers = {}
            for j in idx:
                if j == i:
                    continue
                try:
                    st = nvml.nvmlDeviceGetP2PStatus(h, handles[j], nvml.NVML_P2P_CAPS_INDEX_NVLINK)
                    peers[j] = st == nvml.NVML_P2P_STATUS_OK
                except Exception:  # noqa: BLE001
                    peers[j] = False
            out.append(GpuMemory(i, _text(nvml.nvmlDeviceGetName(h)), int(mem.total), int(mem.free), bar_total,
                                 bar_free, links, peers))
        return out
    finally:
        if own:
            nvml.nvmlShutdown()


def describe(gpus: List[GpuMemory]) -> List[str]:
    """The lines the CLI prints at start-up."""
    lines = []
    for g in gpus:
        peers = ""
        if g.peers_nvlink:
            ok = [str(j) for j, v in sorted(g.peers_nvlink.items()) if v]
            bad = [str(j) for j, v in sorted(g.peers_nvlink.items()) if not v]
            peers = f", NVLink peers [{' '.join(ok)}]" + (f", NOT over NVLink [{' '.join(bad)}]" if bad else "")
        lines.append(f"memory: GPU {g.index} {g.name}: {g.free / 2**30:.1f} of {g.total / 2**30:.1f} GiB free, "
                     f"BAR1 {g.bar1_total / 2**30:.1f} GiB"
                     f"{' (covers the memory)' if g.bar1_covers_memory else ''}, {g.nvlinks_up} NVLinks up{peers}")
    return lines


def check_placement(gpus: List[GpuMemory], need_bytes: int = 0, need_nvlink: bool = False) -> List[str]:
    """Problems of a placement over ``gpus`` (empty list: fine): too little free memory for ``need_bytes`` per
    GPU; with ``need_nvlink`` a pair that is not connected by NVLink."""
    problems = []
    for g in gpus:
        if need_bytes and g.free < need_bytes:
            problems.append(f"GPU {g.index}: {g.free / 2**30:.1f} GiB free, {need_bytes / 2**30:.1f} GiB needed")
        if need_nvlink:
            for j, ok in sorted(g.peers_nvlink.items()):
                if not ok:
                    problems.append(f"GPU {g.index} and GPU {j} are not connected by NVLink")
    return problems
