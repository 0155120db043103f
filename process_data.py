"""Entry point with the reference's name: ``python process_data.py --input-file ... --output-file ...``."""
from mini_trainer_b200.cli.process_data import app

if __name__ == "__main__":
    app()
