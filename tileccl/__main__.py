import sys

from tileccl_b200.cli import main

sys.exit(main())
