"""Serving scheduler. The core (allocator, prefix index, continuous batcher, policy) is C++
(``csrc/sched``); this package re-exports it and adds the Python-level memory tiers and observers."""
from .._lib_loader import load_ext

_sched = load_ext("_sched", "sched")

BlockAllocator = _sched.BlockAllocator
PrefixIndex = _sched.PrefixIndex
SamplingParams = _sched.SamplingParams
PolicyConfig = _sched.PolicyConfig
SystemState = _sched.SystemState
ContinuousBatcher = _sched.ContinuousBatcher
StepPlan = _sched.StepPlan
policy_decide = _sched.policy_decide

SEQ_STATES = {0: "waiting", 1: "prefilling", 2: "running", 3: "paused", 4: "finished"}
FINISH_REASONS = {0: "none", 1: "eos", 2: "length", 3: "aborted", 4: "veto"}
ORDER_STRICT_REQUEST_ID, ORDER_FIFO = 0, 1
