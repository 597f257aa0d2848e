"""Plain reference implementation used by the tests; independent of the product package."""
