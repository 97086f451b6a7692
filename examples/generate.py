#!/usr/bin/env python3
"""Generate with a model folder (or seeded random weights) and show prefix-cache reuse.

    python examples/generate.py --model DIR [--max-tokens 32] [--prompt-ids "1,2,3;4,5,6"]

See ``mini_engine_b200/cli/generate.py`` for every option.
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from mini_engine_b200.cli.generate import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
