"""Import-path compatibility with the reference: `penny.custom_all_reduce`,
`penny.utils` (the implementation lives in penny_b200)."""
