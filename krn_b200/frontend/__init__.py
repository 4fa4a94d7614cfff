"""The typed, signature-only kernel surface of the tile path (names and meanings as in the reference's
`krn.frontend`): dtypes, tensor annotations, records, launch geometry and the device functions a tile kernel calls."""
