"""Runtime counters as metrics.

``snapshot()`` returns ``bf.runtime_stats()`` with the rank attached; ``start_prometheus_exporter(port)`` serves the same
counters (and, on GPU ranks, the device memory in use) in the Prometheus text format from a background HTTP thread, one
exporter per rank (``port + rank``), when the ``prometheus_client`` package is installed.  Scraping reads atomics and
never touches the GPU stream, so it can run beside training.  The reference has no metrics endpoint; its observability
is the log and the timeline (bluefog/common/logging.cc, bluefog/common/timeline.cc).
"""
from typing import Dict, Optional

import torch

from bluefog_b200.common.basics import get_basics

_b = get_basics()
_PREFIX = "bluefog_b200_"


def snapshot() -> Dict[str, int]:
    """The counters of this rank, plus ``rank`` and ``size``."""
    stats = dict(_b.runtime_stats())
    stats["rank"], stats["size"] = _b.rank(), _b.size()
    return stats


def _metric_name(key: str) -> str:
    return _PREFIX + key.lower().replace(".", "_")


class _Collector:
    """prometheus_client custom collector: one counter per entry of the snapshot, labelled with the rank."""

    def collect(self):
        from prometheus_client.core import CounterMetricFamily, GaugeMetricFamily
        try:
            stats = snapshot()
        except Exception:       # not initialised (yet, or any more): nothing to report
            return
        rank = str(stats.pop("rank"))
        stats.pop("size", None)
        per_type = CounterMetricFamily(_PREFIX + "operations_enqueued", "operations enqueued, by type", labels=["rank", "type"])
        for key, value in sorted(stats.items()):
            if key.startswith("enqueued."):
                per_type.add_metric([rank, key.split(".", 1)[1].lower()], value)
            else:
                c = CounterMetricFamily(_metric_name(key), key.replace("_", " "), labels=["rank"])
                c.add_metric([rank], value)
                yield c
        yield per_type
        if torch.cuda.is_available() and _b.device() >= 0:
            g = GaugeMetricFamily(_PREFIX + "device_memory_allocated_bytes", "bytes held by PyTorch's allocator on this rank's GPU",
                                  labels=["rank"])
            g.add_metric([rank], torch.cuda.memory_allocated(_b.device()))
            yield g


def start_prometheus_exporter(port: int = 9400, addr: str = "127.0.0.1", registry=None) -> Optional[int]:
    """Starts the HTTP exporter of this rank on ``port + rank`` and returns that port; None when ``prometheus_client``
    is not installed.  Pass a ``CollectorRegistry`` to register the collector without the default process metrics."""
    try:
        import prometheus_client
    except ImportError:
        return None
    reg = registry if registry is not None else prometheus_client.REGISTRY
    reg.register(_Collector())
    real_port = port + (_b.rank() if _b.is_initialized() else 0)
    prometheus_client.start_http_server(real_port, addr=addr, registry=reg)
    return real_port
