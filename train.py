"""Entry point kept at the repository root so `torchrun ... train.py <flags>` works as in
the reference project; the implementation lives in ``nsa_optim_b200/train.py``."""
from nsa_optim_b200.train import main

if __name__ == "__main__":
    main()
