"""Import path of the reference's `scripts` package (its tests import `scripts.sweep`)."""
