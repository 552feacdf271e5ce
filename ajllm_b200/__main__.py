"""``python -m ajllm_b200`` runs the command-line interface (reference: ``ajllm/__main__.py:1-6``)."""

from ajllm_b200.cli import main

if __name__ == "__main__":
    main()
