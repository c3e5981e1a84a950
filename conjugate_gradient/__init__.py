"""Import-name compatibility with the reference's `conjugate_gradient` package."""
