"""B200 (sm_100a) first-order scan with the reference's drop-in API:
`accelerated_scan.warp.scan(gates, tokens)` and
`accelerated_scan.complex.scan(forget, inputs)`."""
__version__ = "0.1.0"
