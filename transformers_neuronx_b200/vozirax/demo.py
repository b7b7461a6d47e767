"""vozirax_demo: the demo command line (save a folder of random weights from a config.json; load a folder and
sample) for the Vozirax decoder.  Same options as opt_demo; the entry-point class is chosen by config.json."""
from ..opt.demo import main

if __name__ == "__main__":
    main()
