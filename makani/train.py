"""`python -m makani.train`: the upstream command name for `python -m makani_b200.train` (same flags)."""

from makani_b200.train import main

if __name__ == "__main__":
    main()
