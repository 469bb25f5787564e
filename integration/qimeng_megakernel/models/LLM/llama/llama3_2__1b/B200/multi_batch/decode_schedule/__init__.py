"""B200 decode schedule of Llama-3.2-1B (several sequences per step): the compiled route is libqmk_b200.so, whose kernel owns its scheduler and
dependency tracking.  Attributes are what qimeng_megakernel/models/LLM/registry.py:238-262 (import_decode_schedule)
and decode.py:600-642 read from a decode-schedule package."""
from qimeng_megakernel_b200 import Globals, LlamaConfig, ModelConfig  # noqa: F401  (same fields as the A100 Globals)
# the PyTorch routes are shared with the A100 package, as the reference's own multi-batch package does
from qimeng_megakernel.models.LLM.llama.llama3_2__1b.A100.single_batch.decode_schedule.fused import layer_scheduler  # noqa: F401,E402

# decode.py:609-642 skips queue building and tensorising, 688-689 / 1383-1384 skip barriers.zero_()
STATIC_MEGAKERNEL = True
HARDWARE = "B200"
