* s27 (s27 itself: three flip-flops, ten gates): 10 gates, 42 transistors
VDD vdd 0 DC 1.8
VIN0 nG0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 nG1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 nG2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 nG3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 nG5 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 nG6 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 nG7 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
M1 nG14 nG0 vdd vdd pch w=2u l=180n
M2 nG14 nG0 0 0 nch w=1u l=180n
CnG14 nG14 0 2f
M3 nG17 nG11 vdd vdd pch w=2u l=180n
M4 nG17 nG11 0 0 nch w=1u l=180n
CnG17 nG17 0 2f
CT1 t1 0 0.1f
M5 t1 nG14 vdd vdd pch w=2u l=180n
M6 t1 nG6 vdd vdd pch w=2u l=180n
CT2 t2 0 0.1f
M7 t1 nG14 t2 0 nch w=1u l=180n
M8 t2 nG6 0 0 nch w=1u l=180n
M9 nG8 t1 vdd vdd pch w=2u l=180n
M10 nG8 t1 0 0 nch w=1u l=180n
CnG8 nG8 0 2f
CT3 t3 0 0.1f
M11 t3 nG12 0 0 nch w=1u l=180n
M12 t3 nG8 0 0 nch w=1u l=180n
CT4 t4 0 0.1f
M13 t4 nG12 vdd vdd pch w=2u l=180n
M14 t3 nG8 t4 vdd pch w=2u l=180n
M15 nG15 t3 vdd vdd pch w=2u l=180n
M16 nG15 t3 0 0 nch w=1u l=180n
CnG15 nG15 0 2f
CT5 t5 0 0.1f
M17 t5 nG3 0 0 nch w=1u l=180n
M18 t5 nG8 0 0 nch w=1u l=180n
CT6 t6 0 0.1f
M19 t6 nG3 vdd vdd pch w=2u l=180n
M20 t5 nG8 t6 vdd pch w=2u l=180n
M21 nG16 t5 vdd vdd pch w=2u l=180n
M22 nG16 t5 0 0 nch w=1u l=180n
CnG16 nG16 0 2f
M23 nG9 nG16 vdd vdd pch w=2u l=180n
M24 nG9 nG15 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M25 nG9 nG16 t7 0 nch w=1u l=180n
M26 t7 nG15 0 0 nch w=1u l=180n
CnG9 nG9 0 2f
M27 nG10 nG14 0 0 nch w=1u l=180n
M28 nG10 nG11 0 0 nch w=1u l=180n
CT8 t8 0 0.1f
M29 t8 nG14 vdd vdd pch w=2u l=180n
M30 nG10 nG11 t8 vdd pch w=2u l=180n
CnG10 nG10 0 2f
M31 nG11 nG5 0 0 nch w=1u l=180n
M32 nG11 nG9 0 0 nch w=1u l=180n
CT9 t9 0 0.1f
M33 t9 nG5 vdd vdd pch w=2u l=180n
M34 nG11 nG9 t9 vdd pch w=2u l=180n
CnG11 nG11 0 2f
M35 nG12 nG1 0 0 nch w=1u l=180n
M36 nG12 nG7 0 0 nch w=1u l=180n
CT10 t10 0 0.1f
M37 t10 nG1 vdd vdd pch w=2u l=180n
M38 nG12 nG7 t10 vdd pch w=2u l=180n
CnG12 nG12 0 2f
M39 nG13 nG2 0 0 nch w=1u l=180n
M40 nG13 nG12 0 0 nch w=1u l=180n
CT11 t11 0 0.1f
M41 t11 nG2 vdd vdd pch w=2u l=180n
M42 nG13 nG12 t11 vdd pch w=2u l=180n
CnG13 nG13 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nG17 nG10 nG11 nG13
.end
