"""``python -m ttt.generate`` == ``python -m dttt_b200.generate``."""
import sys

from dttt_b200.generate import *  # noqa: F401,F403
from dttt_b200.generate import main

if __name__ == "__main__":
    sys.exit(main())
