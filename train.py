"""Entry point with the reference's name: ``torchrun --nproc-per-node=N train.py --output-dir ...``."""
from mini_trainer_b200.cli.train import app

if __name__ == "__main__":
    app()
