"""Which builds of each source exist: a source may be compiled several times with different -D flags
(for instance one attention kernel per head size).  `all_variants(source)` lists the flag sets that the
build check compiles; at run time only what the loaded model needs is built."""
from typing import List, Tuple

VARIANTS = {
    # one build per head size that the tensor-core attention kernels take
    "attention_mma.cu": [(f"LMSF_HEAD_DIM={hd}",) for hd in range(16, 129, 16)],
    "attention_tc.cu": [("LMSF_HEAD_DIM=64",), ("LMSF_HEAD_DIM=128",)],
}


def all_variants(source: str) -> List[Tuple[str, ...]]:
    return VARIANTS.get(source, [()])
