"""Speculative decoding: draft trees, verification, draft heads, controllers."""
from .engine import AcceptanceController, SelfSpeculativeDecoder, SpecDecodingState, SpecMode  # noqa: F401
from .heads import DraftAdapter, EagleHead, MtpHead, SpeculationCache  # noqa: F401
from .mtp_executor import MtpExecutor, parse_step_tokens  # noqa: F401
from .tree import NgramIndex, SpecTree, tree_attention_mask_csr, tree_attention_mask_dense  # noqa: F401
from .verify import (KvCommitInstruction, KvOp, check_eqspec_invariants, generate_kv_commit_instructions,  # noqa: F401
                     verify_greedy, verify_stochastic, verify_tree_greedy)
