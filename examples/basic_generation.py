"""Minimal usage example: generate with the offline LLM API.

    python examples/basic_generation.py --model DIR --prompt "Explain KV caching briefly."
    python examples/basic_generation.py --model DIR --prompt-len 32 --temperature 0
"""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from tokamak_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
