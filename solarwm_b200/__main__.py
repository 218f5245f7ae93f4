"""``python -m solarwm_b200 <command> ...``: train / infer / preencode / config / data / environment /
publish-validation through the same parser as ``solarwm_b200.cli.main``."""
import sys

from solarwm_b200.cli import main

if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
