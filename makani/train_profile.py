"""`python -m makani.train_profile`: the upstream command name for `python -m makani_b200.train_profile` (same flags)."""

from makani_b200.train_profile import main

if __name__ == "__main__":
    main()
