"""Where the reference checkout is, for the scripts that build checkers from it.

TEST INFRASTRUCTURE ONLY. The location comes from the environment variable
``LOOM_REFERENCE_ROOT``; without it, a directory named ``reference`` beside this
repository is tried. ``None`` means there is no checkout on this machine (the
case on a GPU box, which only uses what was built before).
"""

from __future__ import annotations

import os

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root() -> str | None:
    chosen = os.environ.get("LOOM_REFERENCE_ROOT")
    if chosen:
        return chosen if os.path.isdir(chosen) else None
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return beside if os.path.isdir(beside) else None
