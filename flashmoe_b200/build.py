"""`python -m flashmoe_b200.build [-f] [-v]`: compile libflashmoe_b200.so in-tree for sm_100a."""
import sys

from ._native import build

if __name__ == "__main__":
    print(build(force="-f" in sys.argv, verbose="-v" in sys.argv))
