"""Which builds of each source exist: a source may be compiled several times with different -D flags
(for instance one attention kernel per head size).  `all_variants(source)` lists the flag sets that the
build check compiles; at run time only what the loaded model needs is built."""
from typing import List, Tuple

VARIANTS = {}


def all_variants(source: str) -> List[Tuple[str, ...]]:
    return VARIANTS.get(source, [()])
