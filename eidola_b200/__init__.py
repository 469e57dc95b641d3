"""eidola_b200 -- host-side mirror of libeidola_b200's C ABI (sm_100a decode-step kernels).

The product is the shared library built from eidola_b200/csrc; this package only binds it
(ctypes) for the tests and the benchmark.  Importing it without the built library raises.
"""
from . import capi  # noqa: F401  (fails loudly when the CUDA library is missing)
from .capi import DeviceBuffer, EbError, Timer, device_count, device_info, status_read  # noqa: F401
from .capi import Config, make_config  # noqa: F401
from .host import Comm, Engine, PeerLost, Scheduler, StepGuard, attn_plan, attn_plan_sm_count, kv_append, attn_paged_sink  # noqa: F401
