"""``python -m ttt.data`` == ``python -m dttt_b200.data``."""
import sys

from dttt_b200.data.prep import main

if __name__ == "__main__":
    sys.exit(main())
