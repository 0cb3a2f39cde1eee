"""CPU oracle of the tile-centre render path.  Test infrastructure: never imported by the product."""
