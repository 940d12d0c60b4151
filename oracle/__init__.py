"""CPU oracle for the scan hot path.  Test infrastructure only: the product
package never imports this."""
