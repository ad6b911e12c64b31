"""Entry point kept at the repository root so that ``python main.py <flags>`` works as it does for
the reference (same flags; see ``renee_b200/cli.py``)."""
from renee_b200.cli import main

if __name__ == "__main__":
    main()
