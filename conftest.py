"""Makes `import xma` resolve to the in-tree package (its directory name is not importable)."""

import os
import sys

_ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(_ROOT, "flash-model-architectures_b200"), _ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)
