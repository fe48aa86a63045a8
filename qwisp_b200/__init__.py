"""qwisp_b200 -- B200 (sm_100a) Seedless decode core behind the reference's engine interface.

The package is a thin host-side mirror of the interface qwisp's Tell runtime drives
(`Tell.SpecBackend`, swift/Sources/QwispCore/TellRuntime.swift:83-111) over the C ABI of
libseedless_b200.so (include/seedless_b200.h).  All arithmetic runs in hand-written CUDA
kernels; there is no CPU path and importing the library without it built fails loudly.
"""
from ._lib import SeedlessError, config, lib, synth_spec  # noqa: F401
from .engine import Engine, Stream, SpecBackend, LaneBatchSlots, LaneAdmitPlan, admit_plan  # noqa: F401
from . import ops  # noqa: F401
from . import checkpoint  # noqa: F401
from . import scheduler  # noqa: F401
from .scheduler import ContinuousScheduler, Request  # noqa: F401
from .prefix import PrefixRAMStore, PrefixDiskStore  # noqa: F401
