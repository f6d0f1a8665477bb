"""`python -m makani.inference`: the upstream command name for `python -m makani_b200.inference` (same flags)."""

from makani_b200.inference import main

if __name__ == "__main__":
    main()
